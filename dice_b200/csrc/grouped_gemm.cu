// Grouped (per-expert-segment) GEMM on the sm_100a tensor cores.
//
//   out[r, :] = epilogue( a[r, :] * w[slab(segment(r))]^T )
//
// A persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      loader: one lane issues TMA tile loads (128B-swizzled, K-major)
//               into a 4-deep shared-memory ring;
//   warp 1      tensor-core warp: allocates tensor memory, one lane issues
//               tcgen05.mma (128 x N x 16, bf16 in, fp32 accumulate in tensor
//               memory) and commits ring slots / accumulators to mbarriers;
//   warps 2..5  epilogue: tcgen05.ld the accumulator (one 32-lane quadrant
//               each), apply the activation in fp32, store bf16 rows.
// Two 256-column accumulators alternate, so the epilogue of tile i overlaps
// the main loop of tile i+1.
//
// Raggedness: segments start at arbitrary rows.  The tile list is derived on
// the device from the segment offsets (no host synchronisation): m-blocks are
// counted per segment, a tile's rows start at seg_start + 128*j, the loads may
// run past the segment end (into the next segment or the zero-filled region
// past the last row) and the epilogue stores only the rows that belong to the
// segment.
//
// Every mbarrier wait is bounded by wall time; when one expires the kernel
// records a status code, all roles leave their loops, tensor memory is freed
// and the kernel returns.
#include <stdlib.h>

#include "select.cuh"
#include "umma.cuh"

using namespace dice_umma;

namespace {

// ---- the kernel -------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* aux = smem + kStages * kStageBytes;
  // a narrow weight box leaves room for a deeper ring in the same shared memory
  const uint32_t stage_bytes = kTileABytes + ((static_cast<uint32_t>(p.b_box_rows) * (BK * 2) + 1023u) & ~1023u);
  const int n_stages = p.n_stages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(aux);
  const uint32_t full_bar = smem_u32(bars);                       // [kMaxStages]
  const uint32_t empty_bar = smem_u32(bars + kMaxStages);         // [kMaxStages]
  const uint32_t acc_full_bar = smem_u32(bars + 2 * kMaxStages);  // [kAccStages]
  const uint32_t acc_empty_bar = smem_u32(bars + 2 * kMaxStages + kAccStages);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 2 * kAccStages);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  int* s_seg_off = reinterpret_cast<int*>(tmem_slot + 4);         // [n_seg + 1]
  int* s_mprefix = s_seg_off + (kMaxSeg + 1);                     // [n_seg + 1] m-blocks before segment s
  const uint32_t tiles_smem = smem_u32(smem);
  const uint32_t stage_tx_bytes = kTileABytes + static_cast<uint32_t>(p.b_box_rows) * (BK * 2);
  int* s_hist = s_mprefix + (kMaxSeg + 1);                        // [64] router histogram of this CTA's tiles
  int* s_tile_hist = s_hist + 64;                                 // [kAccStages][64] histogram of the tile in flight

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Set-up that needs no global memory comes first: with a programmatic dependent launch this part overlaps the
  // tail of the kernel before this one in the stream.
  pdl_trigger();
  if (threadIdx.x < 64) s_hist[threadIdx.x] = 0;
  if (threadIdx.x < 64 * kAccStages) s_tile_hist[threadIdx.x] = 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < n_stages; ++s) {
      mbar_init(full_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, 1);
    }
    for (int a = 0; a < kAccStages; ++a) {
      mbar_init(acc_full_bar + 8 * a, 1);
      mbar_init(acc_empty_bar + 8 * a, kEpilogueWarps);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), kTmemCols);
  pdl_wait();  // results of earlier kernels (segment table, rows) are visible from here on

  // a null offset table means one segment covering all rows
  for (int i = threadIdx.x; i <= p.n_seg; i += kThreads)
    s_seg_off[i] = p.seg_offsets != nullptr ? p.seg_offsets[i] : (i == 0 ? 0 : p.n_rows);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    bool ok = s_seg_off[0] >= 0;
    for (int s = 0; s < p.n_seg; ++s) {
      const int cnt = s_seg_off[s + 1] - s_seg_off[s];
      ok = ok && cnt >= 0;
      s_mprefix[s] = run;
      const bool has_weights = p.seg_slab == nullptr || p.seg_slab[s] >= 0;  // slab -1: rows that belong to no expert
      run += (cnt > 0 && has_weights) ? (cnt + BM - 1) / BM : 0;
    }
    ok = ok && s_seg_off[p.n_seg] <= p.n_rows;
    if (!ok) {
      run = 0;
      if (p.status != nullptr) atomicCAS(p.status, 0u, DICE_STATUS_BAD_SEGMENTS);
    }
    s_mprefix[p.n_seg] = run;
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  const uint32_t tmem_base = *tmem_slot;
  const int total_mblk = s_mprefix[p.n_seg];
  const int64_t total_tiles = static_cast<int64_t>(total_mblk) * p.n_nblk;

  if (warp == 0) {
    // ---------------- loader (warp-wide loop, one elected lane issues the copies) ----------------
    {
      // (tile, k-block) cursor over this CTA's share of the tile list
      struct Cursor { int64_t t; int kb, seg, row0, wrow0; bool valid; };
      auto decode = [&](Cursor& c) {
        c.valid = c.t < total_tiles;
        if (!c.valid) return;
        const int mb = static_cast<int>(c.t / p.n_nblk);
        const int nb = static_cast<int>(c.t - static_cast<int64_t>(mb) * p.n_nblk);
        while (mb >= s_mprefix[c.seg + 1]) ++c.seg;
        c.row0 = s_seg_off[c.seg] + (mb - s_mprefix[c.seg]) * BM;
        const int slab = p.seg_slab != nullptr ? p.seg_slab[c.seg] : c.seg;
        c.wrow0 = slab * p.w_rows + nb * BN;
      };
      auto advance = [&](Cursor& c) {
        if (++c.kb == p.n_kblk) { c.kb = 0; c.t += gridDim.x; decode(c); }
      };
      Cursor cur{static_cast<int64_t>(blockIdx.x), 0, 0, 0, 0, false};
      decode(cur);
      int stage = 0;
      uint32_t phase = 0;
      while (cur.valid) {
        if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag, p.status, DICE_STATUS_WAIT_SMEM_EMPTY)) break;
        const uint32_t a_dst = tiles_smem + stage * stage_bytes;
        if (elect_one()) {
          mbar_expect_tx(full_bar + 8 * stage, stage_tx_bytes);
          tma_load_2d(a_dst, &tm_a, cur.kb * BK, cur.row0, full_bar + 8 * stage);
          tma_load_2d(a_dst + kTileABytes, &tm_b, cur.kb * BK, cur.wrow0, full_bar + 8 * stage);
        }
        __syncwarp();
        if (++stage == n_stages) { stage = 0; phase ^= 1u; }
        advance(cur);
      }
    }
  } else if (warp == 1) {
    // ---------------- tensor-core issue (warp-wide loop, one elected lane issues) ----------------
    {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool alive = true;
      for (int64_t t = blockIdx.x; alive && t < total_tiles; t += gridDim.x) {
        const int nb = static_cast<int>(t % p.n_nblk);
        int n_valid = p.w_rows - nb * BN;
        if (n_valid > BN) n_valid = BN;
        const uint32_t idesc = make_instr_desc(BM, (n_valid + 15) & ~15);
        if (!mbar_wait(acc_empty_bar + 8 * acc, acc_phase ^ 1u, abort_flag, p.status, DICE_STATUS_WAIT_ACC_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < p.n_kblk; ++kb) {
          if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag, p.status, DICE_STATUS_WAIT_SMEM_FULL)) {
            alive = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = tiles_smem + stage * stage_bytes;
          const uint64_t a_desc = make_operand_desc(a_addr);
          const uint64_t b_desc = make_operand_desc(a_addr + kTileABytes);
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk) {
              // advance both operands by 16 elements (32 bytes) along K inside the swizzled row
              umma_bf16(d_tmem, a_desc + static_cast<uint64_t>(kk * 2), b_desc + static_cast<uint64_t>(kk * 2), idesc,
                        static_cast<uint32_t>((kb | kk) != 0));
            }
            umma_commit(empty_bar + 8 * stage);  // slot reusable once these MMAs have read it
          }
          __syncwarp();
          if (++stage == n_stages) { stage = 0; phase ^= 1u; }
        }
        if (!alive) break;
        if (elect_one()) umma_commit(acc_full_bar + 8 * acc);   // accumulator complete
        __syncwarp();
        if (++acc == kAccStages) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int quad = warp & 3;            // tensor-memory lanes [32*quad, 32*quad+32) belong to this warp
    const int half = (warp - 2) >> 2;     // which of the quadrant's two warps: even or odd 32-column chunks
    int acc = 0, seg = 0;
    uint32_t acc_phase = 0;
    for (int64_t t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      const int mb = static_cast<int>(t / p.n_nblk);
      const int nb = static_cast<int>(t - static_cast<int64_t>(mb) * p.n_nblk);
      while (mb >= s_mprefix[seg + 1]) ++seg;
      const int row0 = s_seg_off[seg] + (mb - s_mprefix[seg]) * BM;
      const int rows_valid = s_seg_off[seg + 1] - row0;  // may exceed BM
      if (!mbar_wait(acc_full_bar + 8 * acc, acc_phase, abort_flag, p.status, DICE_STATUS_WAIT_ACC_FULL)) break;
      tc_fence_after_sync();
      const int r = quad * 32 + lane;
      const bool row_ok = r < rows_valid;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * BN);
      __nv_bfloat16* out_row = p.out + static_cast<int64_t>(row0 + r) * p.ld_out;
      if (p.epilogue == kEpiRouter) {
        if (half == 0) {
        // one thread = one token: its logits are the first n_experts accumulator columns of its lane
        const int64_t tok = row0 + r;
        int i0 = 0, i1 = 1;
        float p0 = 0.f, p1 = 0.f;
        if (p.n_experts <= 32) {
          uint32_t a[32];
          tmem_ld32(taddr, a);
          tmem_ld_wait();
          float l[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) l[e] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(a[e])));
          if (row_ok && p.logits_out != nullptr) {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (e < p.n_experts) p.logits_out[tok * p.n_experts + e] = __float2bfloat16_rn(l[e]);
          }
          if (p.n_experts <= 8) select_top2<8>(reinterpret_cast<const float(&)[8]>(l), p.n_experts, p.renorm, i0, i1, p0, p1);
          else if (p.n_experts <= 16) select_top2<16>(reinterpret_cast<const float(&)[16]>(l), p.n_experts, p.renorm, i0, i1, p0, p1);
          else select_top2<32>(l, p.n_experts, p.renorm, i0, i1, p0, p1);
        } else {
          uint32_t a[32], b[32];
          tmem_ld32(taddr, a);
          tmem_ld32(taddr + 32, b);
          tmem_ld_wait();
          float l[64];
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            l[e] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(a[e])));
            l[32 + e] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(b[e])));
          }
          if (row_ok && p.logits_out != nullptr) {
#pragma unroll
            for (int e = 0; e < 64; ++e)
              if (e < p.n_experts) p.logits_out[tok * p.n_experts + e] = __float2bfloat16_rn(l[e]);
          }
          select_top2<64>(l, p.n_experts, p.renorm, i0, i1, p0, p1);
        }
        if (row_ok) {
          longlong2 iv; iv.x = i0; iv.y = i1;
          *reinterpret_cast<longlong2*>(p.out_idx + 2 * tok) = iv;
          *reinterpret_cast<float2*>(p.out_w + 2 * tok) = make_float2(p0, p1);
          atomicAdd(&s_tile_hist[acc * 64 + i0], 1);
          atomicAdd(&s_tile_hist[acc * 64 + i1], 1);
        }
        // the four selecting warps meet (named barrier 1), then one thread per expert files the tile's histogram
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int e = quad * 32 + lane;
        if (e < p.n_experts) {
          const int cnt = s_tile_hist[acc * 64 + e];
          if (p.chunk_hist != nullptr) p.chunk_hist[t * p.n_experts + e] = cnt;
          s_hist[e] += cnt;
          s_tile_hist[acc * 64 + e] = 0;
        }
        }
      } else if (p.epilogue == DICE_EPI_SWIGLU) {
        const int col0 = nb * (BN / 2);
        int n_valid = p.n_out - col0;
        if (n_valid > BN / 2) n_valid = BN / 2;
        for (int c = half * 32; c < n_valid; c += 64) {
          uint32_t g[32], u[32];
          tmem_ld32(taddr + c, g);
          tmem_ld32(taddr + BN / 2 + c, u);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = silu_f(__uint_as_float(g[j])) * __uint_as_float(u[j]);
          store_row_chunk(out_row + col0 + c, v, n_valid - c, row_ok);
        }
      } else {
        const int col0 = nb * BN;
        int n_valid = p.n_out - col0;
        if (n_valid > BN) n_valid = BN;
        const bool gelu = p.epilogue == DICE_EPI_GELU_TANH;
        for (int c = half * 32; c < n_valid; c += 64) {
          uint32_t a[32];
          tmem_ld32(taddr + c, a);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float f = __uint_as_float(a[j]);
            v[j] = gelu ? gelu_tanh_f(f) : f;
          }
          store_row_chunk(out_row + col0 + c, v, n_valid - c, row_ok);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar + 8 * acc);
      if (++acc == kAccStages) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (p.epilogue == kEpiRouter && p.hist != nullptr && threadIdx.x < p.n_experts && s_hist[threadIdx.x] != 0)
    atomicAdd(&p.hist[threadIdx.x], s_hist[threadIdx.x]);
  if (*abort_flag != 0) {
    // a wait expired: give copies and MMAs still in flight time to land before the CTA's
    // shared and tensor memory are released
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

// ---- host side shared with the CTA-pair kernel ----------------------------------------
namespace dice_umma {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D bf16 tensor [rows, cols] row-major, box = [box_rows, 64 columns], 128-byte swizzle.
int encode_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return DICE_ERR_CUDA;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {BK, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                        elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? DICE_OK : DICE_ERR_CUDA;
}

int sm_count_cached() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached[dev] = n;
  }
  return cached[dev];
}
}  // namespace dice_umma

namespace {

// CTA pairs (256 x 256 tiles) are the default; DICE_GEMM_PAIR=0 selects the one-CTA-per-tile kernel
bool use_cta_pairs() {
  static int cached = -1;
  if (cached < 0) {
    const char* env = getenv("DICE_GEMM_PAIR");
    cached = (env != nullptr && env[0] == '0') ? 0 : 1;
  }
  return cached == 1;
}

int ring_depth(int b_box_rows) {
  const int stage_bytes = kTileABytes + ((b_box_rows * BK * 2 + 1023) & ~1023);
  const int n = (kStages * kStageBytes) / stage_bytes;
  return n > kMaxStages ? kMaxStages : n;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (cudaFuncSetAttribute(grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) !=
        cudaSuccess)
      return 0;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace

extern "C" int dice_grouped_gemm(const void* a, int64_t n_rows, int k_dim, const void* w, int n_slabs, int64_t w_rows,
                                 const int32_t* seg_offsets, const int32_t* seg_slab, int n_seg, int epilogue,
                                 void* out, int64_t ld_out, int n_out, int reserve_sms, uint32_t* status, void* stream) {
  DICE_CHECK_ARG(n_rows >= 0 && k_dim > 0 && n_slabs > 0 && w_rows > 0 && n_seg >= 0 && reserve_sms >= 0, DICE_ERR_ARG);
  DICE_CHECK_ARG(n_seg <= kMaxSeg, DICE_ERR_LIMIT);
  DICE_CHECK_ARG(epilogue == DICE_EPI_STORE || epilogue == DICE_EPI_GELU_TANH || epilogue == DICE_EPI_SWIGLU,
                 DICE_ERR_ARG);
  DICE_CHECK_ARG(k_dim % 8 == 0 && ld_out % 8 == 0 && n_out % 8 == 0 && n_out > 0 && n_out <= ld_out, DICE_ERR_SHAPE);
  if (epilogue == DICE_EPI_SWIGLU)
    DICE_CHECK_ARG(w_rows % 256 == 0 && static_cast<int64_t>(n_out) <= w_rows / 2, DICE_ERR_SHAPE);
  else
    DICE_CHECK_ARG(static_cast<int64_t>(n_out) <= w_rows, DICE_ERR_SHAPE);
  DICE_CHECK_ARG(n_rows < 0x7fffff00LL && static_cast<int64_t>(n_slabs) * w_rows < 0x7fffff00LL, DICE_ERR_LIMIT);
  if (n_rows == 0 || n_seg == 0) return DICE_OK;
  DICE_CHECK_ARG(a && w && seg_offsets && out, DICE_ERR_ARG);
  DICE_CHECK_ARG(dice_aligned16(a) && dice_aligned16(w) && dice_aligned16(out), DICE_ERR_ALIGN);

  if (use_cta_pairs())
    return dice_internal_gemm_pair(a, n_rows, k_dim, w, n_slabs, w_rows, seg_offsets, seg_slab, n_seg, epilogue, out,
                                   ld_out, n_out, reserve_sms, status, static_cast<cudaStream_t>(stream));
  int sms = sm_count();
  if (sms <= 0) return DICE_ERR_CUDA;
  sms = sms - reserve_sms > 1 ? sms - reserve_sms : 1;
  CUtensorMap tm_a, tm_b;
  int rc = encode_map(&tm_a, a, static_cast<uint64_t>(n_rows), static_cast<uint64_t>(k_dim), BM);
  if (rc != DICE_OK) return rc;
  const int b_box_rows = w_rows >= BN ? BN : static_cast<int>((w_rows + 15) / 16 * 16);
  rc = encode_map(&tm_b, w, static_cast<uint64_t>(n_slabs) * static_cast<uint64_t>(w_rows),
                  static_cast<uint64_t>(k_dim), static_cast<uint32_t>(b_box_rows));
  if (rc != DICE_OK) return rc;

  GemmParams p = {};
  p.seg_offsets = seg_offsets;
  p.seg_slab = seg_slab;
  p.n_seg = n_seg;
  p.n_rows = static_cast<int>(n_rows);
  p.n_kblk = (k_dim + BK - 1) / BK;
  p.n_nblk = static_cast<int>((w_rows + BN - 1) / BN);
  p.w_rows = static_cast<int>(w_rows);
  p.n_out = n_out;
  p.epilogue = epilogue;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ld_out = ld_out;
  p.status = status;
  p.b_box_rows = b_box_rows;
  p.n_stages = ring_depth(b_box_rows);
  p.n_experts = 0;
  p.renorm = 0;
  p.out_idx = nullptr;
  p.out_w = nullptr;
  p.hist = nullptr;
  p.chunk_hist = nullptr;
  p.logits_out = nullptr;

  const int64_t max_tiles = ((n_rows + BM - 1) / BM + n_seg) * p.n_nblk;
  const int grid = static_cast<int>(max_tiles < sms ? max_tiles : sms);
  if (dice_launch(grouped_gemm_kernel, dim3(grid), dim3(kThreads), kSmemBytes, static_cast<cudaStream_t>(stream), tm_a, tm_b,
                  p) != cudaSuccess)
    return DICE_ERR_CUDA;
  return cudaGetLastError() == cudaSuccess ? DICE_OK : DICE_ERR_CUDA;
}

// Router on the tensor cores (bf16): logits = x * w_gate^T as one 128 x 16..64 accumulator tile per 128
// tokens, then every epilogue thread selects the top-2 of its own token.
int dice_internal_router_tc(const void* x, const void* w_gate, int64_t n_tokens, int hidden, int n_experts, int renorm,
                            int64_t* out_idx, float* out_w, int32_t* out_hist, int32_t* out_chunk_hist,
                            void* out_logits, uint32_t* status, cudaStream_t stream) {
  const int sms = sm_count();
  if (sms <= 0) return DICE_ERR_CUDA;
  if (n_tokens >= 0x7fffff00LL) return DICE_ERR_LIMIT;
  CUtensorMap tm_a, tm_b;
  const int b_box_rows = (n_experts + 15) / 16 * 16;
  int rc = encode_map(&tm_a, x, static_cast<uint64_t>(n_tokens), static_cast<uint64_t>(hidden), BM);
  if (rc != DICE_OK) return rc;
  rc = encode_map(&tm_b, w_gate, static_cast<uint64_t>(n_experts), static_cast<uint64_t>(hidden),
                  static_cast<uint32_t>(b_box_rows));
  if (rc != DICE_OK) return rc;
  GemmParams p = {};
  p.seg_offsets = nullptr;
  p.seg_slab = nullptr;
  p.n_seg = 1;
  p.n_rows = static_cast<int>(n_tokens);
  p.n_kblk = (hidden + BK - 1) / BK;
  p.n_nblk = 1;
  p.w_rows = n_experts;
  p.n_out = n_experts;
  p.epilogue = kEpiRouter;
  p.out = nullptr;
  p.ld_out = 0;
  p.status = status;
  p.b_box_rows = b_box_rows;
  p.n_stages = ring_depth(b_box_rows);
  p.n_experts = n_experts;
  p.renorm = renorm;
  p.out_idx = out_idx;
  p.out_w = out_w;
  p.hist = out_hist;
  p.chunk_hist = out_chunk_hist;
  p.logits_out = static_cast<__nv_bfloat16*>(out_logits);
  const int64_t tiles = (n_tokens + BM - 1) / BM;
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  if (dice_launch(grouped_gemm_kernel, dim3(grid), dim3(kThreads), kSmemBytes, stream, tm_a, tm_b, p) != cudaSuccess)
    return DICE_ERR_CUDA;
  return cudaGetLastError() == cudaSuccess ? DICE_OK : DICE_ERR_CUDA;
}

extern "C" int dice_grouped_ffn(const void* rows_in, int64_t n_rows, int hidden, int ffn, int act, const void* w1,
                                const void* w2, int n_slabs, const int32_t* seg_offsets, const int32_t* seg_slab,
                                int n_seg, void* inter, void* rows_out, const void* shared_in, int64_t n_shared,
                                int shared_ffn, const void* shared_w1, const void* shared_w2, void* shared_inter,
                                void* shared_out, int reserve_sms, uint32_t* rows_done, void* first_gemm_done,
                                uint32_t* status, void* stream) {
  DICE_CHECK_ARG(act == DICE_ACT_SWIGLU || act == DICE_ACT_GELU_TANH, DICE_ERR_ARG);
  DICE_CHECK_ARG(hidden > 0 && ffn > 0 && reserve_sms >= 0, DICE_ERR_ARG);
  // counting finished blocks of the output is the CTA-pair kernel's; a caller that asked for it waits on the counters
  if (rows_done != nullptr) DICE_CHECK_ARG(use_cta_pairs() && n_rows > 0 && n_seg > 0, DICE_ERR_ARG);
  // the push that follows the second GEMM waits for `first_gemm_done`: only the second GEMM leaves SMs free for it
  DICE_CHECK_ARG(first_gemm_done == nullptr || rows_done != nullptr, DICE_ERR_ARG);
  const int reserve1 = first_gemm_done != nullptr ? 0 : reserve_sms;
  auto mark_first_done = [&]() -> int {
    if (first_gemm_done == nullptr) return DICE_OK;
    return cudaEventRecord(static_cast<cudaEvent_t>(first_gemm_done), static_cast<cudaStream_t>(stream)) == cudaSuccess
               ? DICE_OK
               : DICE_ERR_CUDA;
  };
  if (n_rows > 0 && n_seg > 0) DICE_CHECK_ARG(inter != nullptr, DICE_ERR_ARG);
  const int epi1 = act == DICE_ACT_SWIGLU ? DICE_EPI_SWIGLU : DICE_EPI_GELU_TANH;
  const int64_t w1_rows = act == DICE_ACT_SWIGLU ? dice_w13_rows(ffn) : ffn;
  if (shared_in == nullptr || n_shared == 0) {
    int rc = dice_grouped_gemm(rows_in, n_rows, hidden, w1, n_slabs, w1_rows, seg_offsets, seg_slab, n_seg, epi1, inter,
                               ffn, ffn, reserve1, status, stream);
    if (rc != DICE_OK) return rc;
    if ((rc = mark_first_done()) != DICE_OK) return rc;
    if (rows_done != nullptr) {
      DICE_CHECK_ARG(n_seg <= kMaxSeg && n_rows < 0x7fffff00LL && hidden % 8 == 0 && ffn % 8 == 0, DICE_ERR_LIMIT);
      DICE_CHECK_ARG(w2 && rows_out && dice_aligned16(w2) && dice_aligned16(rows_out), DICE_ERR_ALIGN);
      return dice_internal_gemm_pair(inter, n_rows, ffn, w2, n_slabs, hidden, seg_offsets, seg_slab, n_seg, DICE_EPI_STORE,
                                     rows_out, hidden, hidden, reserve_sms, status, static_cast<cudaStream_t>(stream),
                                     nullptr, nullptr, nullptr, rows_done);
    }
    return dice_grouped_gemm(inter, n_rows, ffn, w2, n_slabs, hidden, seg_offsets, seg_slab, n_seg, DICE_EPI_STORE,
                             rows_out, hidden, hidden, reserve_sms, status, stream);
  }
  // The always-on shared expert rides in the same two launches as one more problem of the tile list
  // (models.py:355-357 runs it as three more linear layers after the routed experts).
  DICE_CHECK_ARG(n_shared > 0 && shared_ffn > 0 && shared_w1 && shared_w2 && shared_inter && shared_out, DICE_ERR_ARG);
  DICE_CHECK_ARG(use_cta_pairs(), DICE_ERR_ARG);  // the one-CTA-per-tile kernel has no second problem
  DICE_CHECK_ARG(hidden % 8 == 0 && ffn % 8 == 0 && shared_ffn % 8 == 0, DICE_ERR_SHAPE);
  DICE_CHECK_ARG(n_seg <= kMaxSeg && n_shared < 0x7fffff00LL && n_rows < 0x7fffff00LL, DICE_ERR_LIMIT);
  DICE_CHECK_ARG(dice_aligned16(shared_in) && dice_aligned16(shared_w1) && dice_aligned16(shared_w2) &&
                     dice_aligned16(shared_inter) && dice_aligned16(shared_out),
                 DICE_ERR_ALIGN);
  const int64_t sw1_rows = act == DICE_ACT_SWIGLU ? dice_w13_rows(shared_ffn) : shared_ffn;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n_rows == 0 || n_seg == 0) {
    // no routed rows on this rank: the shared expert alone, as one segment over all tokens
    int rc = dice_internal_gemm_pair(shared_in, n_shared, hidden, shared_w1, 1, sw1_rows, nullptr, nullptr, 1, epi1,
                                     shared_inter, shared_ffn, shared_ffn, reserve_sms, status, s);
    if (rc != DICE_OK) return rc;
    return dice_internal_gemm_pair(shared_inter, n_shared, shared_ffn, shared_w2, 1, hidden, nullptr, nullptr, 1,
                                   DICE_EPI_STORE, shared_out, hidden, hidden, reserve_sms, status, s);
  }
  DICE_CHECK_ARG(rows_in && w1 && w2 && seg_offsets && rows_out, DICE_ERR_ARG);
  DICE_CHECK_ARG(dice_aligned16(rows_in) && dice_aligned16(w1) && dice_aligned16(w2) && dice_aligned16(inter) &&
                     dice_aligned16(rows_out),
                 DICE_ERR_ALIGN);
  DiceDenseSpec x1 = {shared_in, n_shared, hidden, shared_w1, sw1_rows, shared_inter, shared_ffn, shared_ffn};
  int rc = dice_internal_gemm_pair(rows_in, n_rows, hidden, w1, n_slabs, w1_rows, seg_offsets, seg_slab, n_seg, epi1, inter,
                                   ffn, ffn, reserve1, status, s, nullptr, &x1);
  if (rc != DICE_OK) return rc;
  if ((rc = mark_first_done()) != DICE_OK) return rc;
  DiceDenseSpec x2 = {shared_inter, n_shared, shared_ffn, shared_w2, hidden, shared_out, hidden, hidden};
  return dice_internal_gemm_pair(inter, n_rows, ffn, w2, n_slabs, hidden, seg_offsets, seg_slab, n_seg, DICE_EPI_STORE,
                                 rows_out, hidden, hidden, reserve_sms, status, s, nullptr, &x2, nullptr, rows_done);
}

// The expert FFN whose second GEMM scales every row by its gate weight and adds it to its token's row
// (models.py:377-381) with 16-byte bf16 reductions: no sorted output, no combine kernel.
extern "C" int dice_grouped_ffn_combine(const void* rows_in, int64_t n_rows, int hidden, int ffn, int act,
                                        const void* w1, const void* w2, int n_slabs, const int32_t* seg_offsets,
                                        const int32_t* seg_slab, int n_seg, void* inter, const int32_t* order,
                                        const float* row_weights, int k, void* out_tokens, int reserve_sms,
                                        uint32_t* status, void* stream) {
  DICE_CHECK_ARG(act == DICE_ACT_SWIGLU || act == DICE_ACT_GELU_TANH, DICE_ERR_ARG);
  DICE_CHECK_ARG(n_rows >= 0 && hidden > 0 && ffn > 0 && n_slabs > 0 && n_seg >= 0 && reserve_sms >= 0, DICE_ERR_ARG);
  DICE_CHECK_ARG(k == 2 && n_rows % 2 == 0, DICE_ERR_SHAPE);  // two addends per token: the sum is order-independent
  DICE_CHECK_ARG(hidden % 8 == 0 && ffn % 8 == 0, DICE_ERR_SHAPE);
  DICE_CHECK_ARG(n_seg <= kMaxSeg && n_rows < 0x7fffff00LL, DICE_ERR_LIMIT);
  DICE_CHECK_ARG(use_cta_pairs(), DICE_ERR_ARG);
  if (n_rows == 0) return DICE_OK;
  DICE_CHECK_ARG(rows_in && w1 && w2 && seg_offsets && inter && order && row_weights && out_tokens, DICE_ERR_ARG);
  DICE_CHECK_ARG(dice_aligned16(rows_in) && dice_aligned16(w1) && dice_aligned16(w2) && dice_aligned16(inter) &&
                     dice_aligned16(out_tokens),
                 DICE_ERR_ALIGN);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int epi1 = act == DICE_ACT_SWIGLU ? DICE_EPI_SWIGLU : DICE_EPI_GELU_TANH;
  const int64_t w1_rows = act == DICE_ACT_SWIGLU ? dice_w13_rows(ffn) : ffn;
  DICE_CUDA_OK(cudaMemsetAsync(out_tokens, 0, static_cast<size_t>(n_rows / 2) * hidden * 2, s));
  int rc = dice_grouped_gemm(rows_in, n_rows, hidden, w1, n_slabs, w1_rows, seg_offsets, seg_slab, n_seg, epi1, inter, ffn,
                             ffn, reserve_sms, status, stream);
  if (rc != DICE_OK) return rc;
  if (n_seg == 0) return DICE_OK;
  DiceCombineSpec c = {order, row_weights};
  return dice_internal_gemm_pair(inter, n_rows, ffn, w2, n_slabs, hidden, seg_offsets, seg_slab, n_seg, DICE_EPI_STORE,
                                 out_tokens, hidden, hidden, reserve_sms, status, s, nullptr, nullptr, &c);
}

// The expert FFN whose second GEMM writes its rows straight into the token owners' combine buffers
// (peer memory) and raises their flags when the whole grid is done: FFN + return of the exchange in
// one launch pair.  `out` rows are not stored locally.
extern "C" int dice_grouped_ffn_return(const void* rows_in, int64_t n_rows, int hidden, int ffn, int act,
                                       const void* w1, const void* w2, int n_slabs, const int32_t* seg_offsets,
                                       const int32_t* seg_slab, int n_seg, void* inter, const int32_t* meta,
                                       const void* const* peer_back, const void* const* peer_flags,
                                       uint32_t* done_counter, int rank, int world, int back_capacity_rows,
                                       uint32_t seq, int reserve_sms, uint32_t* status, void* stream) {
  DICE_CHECK_ARG(act == DICE_ACT_SWIGLU || act == DICE_ACT_GELU_TANH, DICE_ERR_ARG);
  DICE_CHECK_ARG(n_rows > 0 && n_seg > 0 && hidden > 0 && ffn > 0 && n_slabs > 0, DICE_ERR_ARG);
  DICE_CHECK_ARG(rows_in && w1 && w2 && seg_offsets && inter && meta && peer_back && peer_flags && done_counter,
                 DICE_ERR_ARG);
  DICE_CHECK_ARG(n_seg <= kMaxSeg && world >= 1 && world <= kMaxPeerRanks && rank >= 0 && rank < world, DICE_ERR_LIMIT);
  DICE_CHECK_ARG(hidden % 8 == 0 && ffn % 8 == 0, DICE_ERR_SHAPE);
  DICE_CHECK_ARG(dice_aligned16(rows_in) && dice_aligned16(w1) && dice_aligned16(w2) && dice_aligned16(inter),
                 DICE_ERR_ALIGN);
  int rc;
  if (act == DICE_ACT_SWIGLU)
    rc = dice_grouped_gemm(rows_in, n_rows, hidden, w1, n_slabs, dice_w13_rows(ffn), seg_offsets, seg_slab, n_seg,
                           DICE_EPI_SWIGLU, inter, ffn, ffn, reserve_sms, status, stream);
  else
    rc = dice_grouped_gemm(rows_in, n_rows, hidden, w1, n_slabs, ffn, seg_offsets, seg_slab, n_seg, DICE_EPI_GELU_TANH,
                           inter, ffn, ffn, reserve_sms, status, stream);
  if (rc != DICE_OK) return rc;
  DiceReturnSpec ret;
  ret.world = world;
  ret.rank = rank;
  ret.capacity_rows = back_capacity_rows;
  ret.meta = meta;
  ret.bufs = peer_back;
  ret.flags = peer_flags;
  ret.done_counter = done_counter;
  ret.seq = seq;
  // `out` is only a base for pointer arithmetic that the return mapping replaces
  return dice_internal_gemm_pair(inter, n_rows, ffn, w2, n_slabs, hidden, seg_offsets, seg_slab, n_seg, DICE_EPI_STORE,
                                 const_cast<void*>(peer_back[rank]), hidden, hidden, reserve_sms, status,
                                 static_cast<cudaStream_t>(stream), &ret);
}
