// Grouped GEMM with CTA pairs (tcgen05 cta_group::2).
//
// Same contract as grouped_gemm.cu, different tiling: two CTAs of a cluster
// share one 256 x 256 tile.  CTA r of the pair loads its own 128 rows of A and
// HALF of the weight tile (128 of the 256 weight rows); one thread of the
// leader CTA issues tcgen05.mma.cta_group::2 (M = 256), which reads A from
// both CTAs' shared memory and stitches the two weight halves together, and
// leaves rows [128 r, 128 r + 128) of the result in CTA r's tensor memory.
// Per SM and k-block that is 32 KB of operands instead of 48 KB, so shared
// memory carries a third less traffic and the same 192 KB ring holds six
// slots instead of four.
//
// Synchronisation across the pair:
//   * both loaders' TMA copies complete on the LEADER's "full" mbarrier (the
//     leader arms it with the pair's byte count);
//   * the leader's MMA thread commits to the "empty" and "accumulator full"
//     mbarriers of BOTH CTAs;
//   * the epilogue warps of both CTAs arrive on the LEADER's "accumulator
//     empty" mbarrier;
//   * a cluster barrier before the exit keeps either CTA alive until its peer
//     can no longer signal it.
// Every wait is bounded as in the single-CTA kernel.
#include <cuda.h>
#include "umma.cuh"

using namespace dice_umma;

namespace {

constexpr int PM = 256;                    // rows per tile pair
constexpr int kPairStages = 6;
constexpr int kPairTileBBytes = 128 * BK * 2;
constexpr int kPairStageBytes = kTileABytes + kPairTileBBytes;  // 32 KB
constexpr int kStoreStageBytes = 2048;  // per epilogue warp: 32 rows x 64 bytes, transposed between the tensor-memory
                                        // layout (one row per lane) and full 64-byte row pieces per store
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + kAuxBytes + kEpilogueWarps * kStoreStageBytes + 1024;

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrival on a barrier of the pair's other CTA with the default (CTA-scope) ordering.  It hands an accumulator
// back, which the tcgen05 fences order; a cluster-scope release would also wait for the warp's global stores.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of this CTA whose completion is counted on the leader's mbarrier
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                                 uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(leader_bar)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot_smem_addr, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem_addr), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive (once all MMAs issued so far have completed) on the mbarrier at this offset in both CTAs of the pair
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(both)
               : "memory");
}

// 16 bytes of bf16 added to global memory (no return value): the combine epilogue's store
__device__ __forceinline__ void red_add_bf16x8(void* dst, const uint4& v) {
  asm volatile("red.relaxed.gpu.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// The loader and the tensor-core warp run their loops with all 32 lanes (the waits are warp-wide) and elect one
// lane for the TMA / MMA instructions: loop state stays warp-uniform for the compiler, and the issue loop is
// short enough to keep the tensor pipe fed (a single-lane loop under `lane == 0` was 15 % slower).
#ifdef DICE_FOLLOW_TRACE
// debug build only: first start and last end of every launch (time stamps of the global timer)
__device__ unsigned long long g_gemm_start[1024];
__device__ unsigned long long g_gemm_end[1024];
#endif

__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                         const __grid_constant__ CUtensorMap tm_b_narrow, const __grid_constant__ CUtensorMap tm_xa,
                         const __grid_constant__ CUtensorMap tm_xb, const __grid_constant__ CUtensorMap tm_xb_narrow,
                         const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* aux = smem + kPairStages * kPairStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(aux);
  const uint32_t full_bar = smem_u32(bars);                          // [kPairStages] used in the leader
  const uint32_t empty_bar = smem_u32(bars + kPairStages);           // [kPairStages] in both CTAs
  const uint32_t acc_full_bar = smem_u32(bars + 2 * kPairStages);    // [kAccStages] in both CTAs
  const uint32_t acc_empty_bar = smem_u32(bars + 2 * kPairStages + kAccStages);  // used in the leader
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kPairStages + 2 * kAccStages);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  int* s_seg_off = reinterpret_cast<int*>(tmem_slot + 4);
  int* s_mprefix = s_seg_off + (kMaxSeg + 1);
  int* s_ret_src = s_mprefix + (kMaxSeg + 1);   // [W + 1] first received row of each source rank
  int* s_ret_base = s_ret_src + (kMaxPeerRanks + 1);  // [W] first row of this rank's block in each source's buffer
  const uint32_t tiles_smem = smem_u32(smem);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_cta_rank();  // 0 = leader
  const bool leader = cta_rank == 0;
  const int64_t pair_id = blockIdx.x >> 1;
  const int64_t n_pairs = gridDim.x >> 1;

  // Set-up that needs no global memory comes first: with a programmatic dependent launch this part overlaps the
  // tail of the kernel before this one in the stream.
  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {  // all slots' barriers exist even when fewer are used
      mbar_init(full_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, 1);
    }
    for (int a = 0; a < kAccStages; ++a) {
      mbar_init(acc_full_bar + 8 * a, 1);
      mbar_init(acc_empty_bar + 8 * a, 2 * kEpilogueWarps);  // the epilogue warps of both CTAs
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
  pdl_wait();  // the segment table and the rows written by earlier kernels are visible from here on
#ifdef DICE_FOLLOW_TRACE
  if (threadIdx.x == 0) {
    unsigned long long now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    atomicMin(&g_gemm_start[p.trace_id & 1023], now);
  }
#endif

  if (p.ret_world > 0) {
    if (threadIdx.x <= p.ret_world) s_ret_src[threadIdx.x] = p.ret_meta[2 + 2 * p.ret_world + threadIdx.x];  // src_off of the meta block
    if (threadIdx.x < p.ret_world) s_ret_base[threadIdx.x] = p.ret_meta[2 + p.ret_world + threadIdx.x];
  }
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
      run += (cnt > 0 && has_weights) ? (cnt + PM - 1) / PM : 0;
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
  cluster_barrier();  // the peer's mbarriers are initialised before anything signals them
  tc_fence_after_sync();

  const uint32_t tmem_base = *tmem_slot;
  // tile list: the segmented problem's tiles, then the tiles of the appended dense problem (if any)
  const int64_t tiles0 = static_cast<int64_t>(s_mprefix[p.n_seg]) * p.n_nblk;
  const int64_t total_tiles = tiles0 + static_cast<int64_t>((p.x_rows + PM - 1) / PM) * p.x_nblk;
  // tile t -> problem (0 / 1), n-block, first row of this CTA's half and the rows that belong to the tile's segment
  struct Tile { int g, nb, row0, rows_valid, slab; };
  auto decode = [&](int64_t t, int& seg) {
    Tile ti;
    if (t < tiles0) {
      const int mb = static_cast<int>(t / p.n_nblk);
      ti.g = 0;
      ti.nb = static_cast<int>(t - static_cast<int64_t>(mb) * p.n_nblk);
      while (mb >= s_mprefix[seg + 1]) ++seg;
      ti.row0 = s_seg_off[seg] + (mb - s_mprefix[seg]) * PM + static_cast<int>(cta_rank) * BM;
      ti.rows_valid = s_seg_off[seg + 1] - ti.row0;  // <= 0 when this CTA's half lies past the segment
      ti.slab = p.seg_slab != nullptr ? p.seg_slab[seg] : seg;
    } else {
      const int64_t t1 = t - tiles0;
      const int mb = static_cast<int>(t1 / p.x_nblk);
      ti.g = 1;
      ti.nb = static_cast<int>(t1 - static_cast<int64_t>(mb) * p.x_nblk);
      ti.row0 = mb * PM + static_cast<int>(cta_rank) * BM;
      ti.rows_valid = p.x_rows - ti.row0;
      ti.slab = 0;
    }
    return ti;
  };

  if (warp == 0) {
    // ---------------- loader (both CTAs) ----------------
    {
      int stage = 0, seg = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int64_t t = pair_id; alive && t < total_tiles; t += n_pairs) {
        const Tile ti = decode(t, seg);
        const int w_rows = ti.g == 0 ? p.w_rows : p.x_w_rows;
        const int n_kblk = ti.g == 0 ? p.n_kblk : p.x_kblk;
        const CUtensorMap* map_a = ti.g == 0 ? &tm_a : &tm_xa;
        const int row0 = ti.row0;
        int n_valid = w_rows - ti.nb * BN;
        if (n_valid > BN) n_valid = BN;
        const int n_mma = (n_valid + 15) & ~15;
        // the MMA takes the first n_mma/2 weight rows of the tile from the leader and the rest from the peer
        const int wrow0 = ti.slab * w_rows + ti.nb * BN + static_cast<int>(cta_rank) * (n_mma / 2);
        // a tile of at most 128 weight rows needs 64 of them per CTA: the narrow box moves half the bytes
        const bool narrow = n_mma <= 128;
        const CUtensorMap* map_b = ti.g == 0 ? (narrow ? &tm_b_narrow : &tm_b) : (narrow ? &tm_xb_narrow : &tm_xb);
        const uint32_t pair_bytes = 2u * (kTileABytes + (narrow ? kPairTileBBytes / 2 : kPairTileBBytes));
        for (int kb = 0; kb < n_kblk; ++kb) {
          if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag, p.status, DICE_STATUS_WAIT_SMEM_EMPTY)) {
            alive = false;
            break;
          }
          const uint32_t a_dst = tiles_smem + stage * kPairStageBytes;
          const uint32_t leader_full = map_to_cta(full_bar + 8 * stage, 0);
          if (elect_one()) {
            if (leader) mbar_expect_tx(full_bar + 8 * stage, pair_bytes);
            tma_load_2d_pair(a_dst, map_a, kb * BK, row0, leader_full);
            tma_load_2d_pair(a_dst + kTileABytes, map_b, kb * BK, wrow0, leader_full);
          }
          __syncwarp();
          if (++stage == p.n_stages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- tensor-core issue (leader only) ----------------
    if (leader) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool alive = true;
      for (int64_t t = pair_id; alive && t < total_tiles; t += n_pairs) {
        const bool first = t < tiles0;
        const int nb = static_cast<int>(first ? t % p.n_nblk : (t - tiles0) % p.x_nblk);
        const int n_kblk = first ? p.n_kblk : p.x_kblk;
        int n_valid = (first ? p.w_rows : p.x_w_rows) - nb * BN;
        if (n_valid > BN) n_valid = BN;
        const uint32_t idesc = make_instr_desc(PM, (n_valid + 15) & ~15);
        if (!mbar_wait(acc_empty_bar + 8 * acc, acc_phase ^ 1u, abort_flag, p.status, DICE_STATUS_WAIT_ACC_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < n_kblk; ++kb) {
          if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag, p.status, DICE_STATUS_WAIT_SMEM_FULL)) {
            alive = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = tiles_smem + stage * kPairStageBytes;
          const uint64_t a_desc = make_operand_desc(a_addr);
          const uint64_t b_desc = make_operand_desc(a_addr + kTileABytes);
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk)
              umma_bf16_pair(d_tmem, a_desc + static_cast<uint64_t>(kk * 2), b_desc + static_cast<uint64_t>(kk * 2), idesc,
                             static_cast<uint32_t>((kb | kk) != 0));
            umma_commit_pair(empty_bar + 8 * stage);
          }
          __syncwarp();
          if (++stage == p.n_stages) { stage = 0; phase ^= 1u; }
        }
        if (!alive) break;
        if (elect_one()) umma_commit_pair(acc_full_bar + 8 * acc);
        __syncwarp();
        if (++acc == kAccStages) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ---------------- epilogue (both CTAs, each over its own 128 rows) ----------------
    const int quad = warp & 3;            // tensor-memory lanes [32*quad, 32*quad+32) belong to this warp
    const int half = (warp - 2) >> 2;     // which of the quadrant's two warps: even or odd 32-column chunks
    int acc = 0, seg = 0;
    uint32_t acc_phase = 0;
    for (int64_t t = pair_id; t < total_tiles; t += n_pairs) {
      const Tile ti = decode(t, seg);
      const int nb = ti.nb, row0 = ti.row0, rows_valid = ti.rows_valid;
      __nv_bfloat16* const out = ti.g == 0 ? p.out : p.x_out;
      const int64_t ld_out = ti.g == 0 ? p.ld_out : p.x_ld_out;
      const int n_out = ti.g == 0 ? p.n_out : p.x_n_out;
      if (!mbar_wait(acc_full_bar + 8 * acc, acc_phase, abort_flag, p.status, DICE_STATUS_WAIT_ACC_FULL)) break;
      tc_fence_after_sync();
      const int r = quad * 32 + lane;
      const bool row_ok = r < rows_valid;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * BN);
      // Stores go through a small per-warp transpose in shared memory: a lane holds 32 columns of ONE row,
      // but a store instruction should cover whole 64-byte row pieces.  After the transpose lane l writes
      // piece (l & 3) of rows (l >> 2) + 8 i, i < 4, whose destinations are resolved once per tile.
      __nv_bfloat16* dst_rows[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int rr = quad * 32 + i * 8 + (lane >> 2);
        const int gr = row0 + rr;
        dst_rows[i] = nullptr;
        if (rr < rows_valid) {
          if (p.epilogue == kEpiCombine) {
            // the row is added to the row of the token it belongs to (two rows per token)
            dst_rows[i] = out + static_cast<int64_t>(p.cmb_order[gr] >> 1) * ld_out;
          } else if (p.ret_world > 0 && ti.g == 0) {
            // the row goes straight into the buffer of the rank whose token it is, over NVLink
            int src = 0;
            while (src + 1 < p.ret_world && gr >= s_ret_src[src + 1]) ++src;
            const int dst_row = s_ret_base[src] + (gr - s_ret_src[src]);
            if (dst_row < p.ret_capacity_rows)
              dst_rows[i] = static_cast<__nv_bfloat16*>(p.ret_bufs[src]) + static_cast<int64_t>(dst_row) * ld_out;
            else if (p.status != nullptr)
              atomicCAS(p.status, 0u, DICE_STATUS_EXCHANGE_OVERFLOW);
          } else {
            dst_rows[i] = out + static_cast<int64_t>(gr) * ld_out;
          }
        }
      }
      // combine epilogue: this lane's own row is scaled by its gate weight before the transpose
      const bool combine = p.epilogue == kEpiCombine;
      float row_weight = 1.f;
      if (combine && row_ok) row_weight = p.cmb_weights[p.cmb_order[row0 + r]];
      uint4* stage = reinterpret_cast<uint4*>(aux + kAuxBytes + (warp - 2) * kStoreStageBytes);
      auto staged_store = [&](const float (&v)[32], int col, int n_left) {
        const int swz = (lane >> 1) & 3;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          stage[lane * 4 + (j ^ swz)] =
              make_uint4(pack_bf16x2(v[8 * j + 0], v[8 * j + 1]), pack_bf16x2(v[8 * j + 2], v[8 * j + 3]),
                         pack_bf16x2(v[8 * j + 4], v[8 * j + 5]), pack_bf16x2(v[8 * j + 6], v[8 * j + 7]));
        __syncwarp();
        const int piece = lane & 3;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int rr = i * 8 + (lane >> 2);
          const uint4 val = stage[rr * 4 + (piece ^ ((rr >> 1) & 3))];
          if (dst_rows[i] != nullptr && piece * 8 < n_left) {
            if (combine) red_add_bf16x8(dst_rows[i] + col + piece * 8, val);
            else *reinterpret_cast<uint4*>(dst_rows[i] + col + piece * 8) = val;
          }
        }
        __syncwarp();
      };
      if (p.epilogue == DICE_EPI_SWIGLU) {
        const int col0 = nb * (BN / 2);
        int n_valid = n_out - col0;
        if (n_valid > BN / 2) n_valid = BN / 2;
        for (int c = half * 32; c < n_valid; c += 64) {
          uint32_t g[32], u[32];
          tmem_ld32(taddr + c, g);
          tmem_ld32(taddr + BN / 2 + c, u);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = silu_f(__uint_as_float(g[j])) * __uint_as_float(u[j]);
          staged_store(v, col0 + c, n_valid - c);
        }
      } else {
        const int col0 = nb * BN;
        int n_valid = n_out - col0;
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
            v[j] = gelu ? gelu_tanh_f(f) : f * row_weight;
          }
          staged_store(v, col0 + c, n_valid - c);
        }
      }
      if (p.rows_done != nullptr && ti.g == 0) {
        __threadfence();  // every lane's stores of this tile are visible device-wide before the block is counted
        __syncwarp();
        if (lane == 0) atomicAdd(&p.rows_done[t / p.n_nblk], 1u);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(acc_empty_bar + 8 * acc, 0));
      if (++acc == kAccStages) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (p.ret_world > 0) {
    // every CTA's stores are out; the last CTA of the grid tells the token owners that their rows have arrived
    __threadfence_system();
    __syncthreads();
    __shared__ int s_last;
    if (threadIdx.x == 0) s_last = atomicAdd(p.ret_done_counter, 1u) == gridDim.x - 1;
    __syncthreads();
    if (s_last) {
      __threadfence_system();
      if (threadIdx.x < p.ret_world)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.ret_flags[threadIdx.x] + p.ret_rank), "r"(p.ret_seq)
                     : "memory");
      if (threadIdx.x == 0) *p.ret_done_counter = 0;
    }
  }
#ifdef DICE_FOLLOW_TRACE
  if (threadIdx.x == 64) {
    unsigned long long now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    atomicMax(&g_gemm_end[p.trace_id & 1023], now);
  }
#endif
  cluster_barrier();  // neither CTA leaves while the other may still signal its mbarriers or read its operands
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// number of CTA pairs that can be resident at once (cached per device); 0 on error
int resident_pairs() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    if (cudaFuncSetAttribute(grouped_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes) !=
        cudaSuccess)
      return 0;
    const int sms = sm_count_cached();
    if (sms <= 0) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(sms & ~1), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = kPairSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, grouped_gemm_pair_kernel, &cfg) != cudaSuccess || n <= 0) return 0;
    cached[dev] = n < sms / 2 ? n : sms / 2;
  }
  return cached[dev];
}

}  // namespace

// Internal entry used by dice_grouped_gemm: same arguments, already validated.
#ifdef DICE_FOLLOW_TRACE
static int g_trace_next = 0;
static int g_trace_kind[1024];
extern "C" __attribute__((visibility("default"))) int dice_debug_gemm_trace(unsigned long long* start, unsigned long long* end,
                                                                            int* kind) {
  cudaDeviceSynchronize();
  const int n = g_trace_next < 1024 ? g_trace_next : 1024;
  if (start != nullptr) {
    cudaMemcpyFromSymbol(start, g_gemm_start, sizeof(unsigned long long) * 1024);
    cudaMemcpyFromSymbol(end, g_gemm_end, sizeof(unsigned long long) * 1024);
    for (int i = 0; i < 1024; ++i) kind[i] = g_trace_kind[i];
  }
  void *ps, *pe;
  cudaGetSymbolAddress(&ps, g_gemm_start);
  cudaGetSymbolAddress(&pe, g_gemm_end);
  cudaMemset(ps, 0xff, sizeof(unsigned long long) * 1024);
  cudaMemset(pe, 0, sizeof(unsigned long long) * 1024);
  g_trace_next = 0;
  return n;
}
#endif

int dice_internal_gemm_pair(const void* a, int64_t n_rows, int k_dim, const void* w, int n_slabs, int64_t w_rows,
                            const int32_t* seg_offsets, const int32_t* seg_slab, int n_seg, int epilogue, void* out,
                            int64_t ld_out, int n_out, int reserve_sms, uint32_t* status, cudaStream_t stream,
                            const DiceReturnSpec* ret, const DiceDenseSpec* extra, const DiceCombineSpec* combine,
                            uint32_t* rows_done) {
  int pairs = resident_pairs();
  if (pairs <= 0) return DICE_ERR_CUDA;
  // SM pairs left to kernels of other streams (the side-stream pushes of the asynchronous exchange)
  pairs -= (reserve_sms + 1) / 2;
  if (pairs < 1) pairs = 1;
  CUtensorMap tm_a, tm_b, tm_b_narrow;
  int rc = encode_map(&tm_a, a, static_cast<uint64_t>(n_rows), static_cast<uint64_t>(k_dim), BM);
  if (rc != DICE_OK) return rc;
  rc = encode_map(&tm_b, w, static_cast<uint64_t>(n_slabs) * static_cast<uint64_t>(w_rows), static_cast<uint64_t>(k_dim),
                  128);
  if (rc != DICE_OK) return rc;
  rc = encode_map(&tm_b_narrow, w, static_cast<uint64_t>(n_slabs) * static_cast<uint64_t>(w_rows),
                  static_cast<uint64_t>(k_dim), 64);
  if (rc != DICE_OK) return rc;
  CUtensorMap tm_xa = tm_a, tm_xb = tm_b, tm_xb_narrow = tm_b_narrow;
  GemmParams p = {};
  if (extra != nullptr && extra->n_rows > 0) {
    rc = encode_map(&tm_xa, extra->a, static_cast<uint64_t>(extra->n_rows), static_cast<uint64_t>(extra->k_dim), BM);
    if (rc != DICE_OK) return rc;
    rc = encode_map(&tm_xb, extra->w, static_cast<uint64_t>(extra->w_rows), static_cast<uint64_t>(extra->k_dim), 128);
    if (rc != DICE_OK) return rc;
    rc = encode_map(&tm_xb_narrow, extra->w, static_cast<uint64_t>(extra->w_rows), static_cast<uint64_t>(extra->k_dim), 64);
    if (rc != DICE_OK) return rc;
    p.x_rows = static_cast<int>(extra->n_rows);
    p.x_kblk = (extra->k_dim + BK - 1) / BK;
    p.x_nblk = static_cast<int>((extra->w_rows + BN - 1) / BN);
    p.x_w_rows = static_cast<int>(extra->w_rows);
    p.x_n_out = extra->n_out;
    p.x_out = static_cast<__nv_bfloat16*>(extra->out);
    p.x_ld_out = extra->ld_out;
  }
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
  p.b_box_rows = 128;
  p.n_stages = kPairStages;
  p.rows_done = rows_done;
#ifdef DICE_FOLLOW_TRACE
  p.trace_id = g_trace_next;
  g_trace_kind[g_trace_next & 1023] = epilogue + (rows_done != nullptr ? 1000 : 0);
  ++g_trace_next;
#endif
  if (combine != nullptr) {
    if (epilogue != DICE_EPI_STORE || ret != nullptr || extra != nullptr || !combine->order || !combine->weights)
      return DICE_ERR_ARG;
    p.epilogue = kEpiCombine;
    p.cmb_order = combine->order;
    p.cmb_weights = combine->weights;
  }
  if (ret != nullptr) {
    if (ret->world < 1 || ret->world > kMaxPeerRanks || epilogue != DICE_EPI_STORE) return DICE_ERR_ARG;
    p.ret_world = ret->world;
    p.ret_rank = ret->rank;
    p.ret_capacity_rows = ret->capacity_rows;
    p.ret_meta = ret->meta;
    p.ret_done_counter = ret->done_counter;
    p.ret_seq = ret->seq;
    for (int i = 0; i < ret->world; ++i) {
      if (ret->bufs[i] == nullptr || ret->flags[i] == nullptr) return DICE_ERR_ARG;
      p.ret_bufs[i] = const_cast<void*>(ret->bufs[i]);
      p.ret_flags[i] = static_cast<uint32_t*>(const_cast<void*>(ret->flags[i]));
    }
  }

  const int64_t max_tiles = ((n_rows + PM - 1) / PM + n_seg) * p.n_nblk + static_cast<int64_t>((p.x_rows + PM - 1) / PM) * p.x_nblk;
  const int use_pairs = static_cast<int>(max_tiles < pairs ? max_tiles : pairs);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(2 * use_pairs), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kPairSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dice_pdl_enabled() ? 2 : 1;
  dice_count_launch();
  if (cudaLaunchKernelEx(&cfg, grouped_gemm_pair_kernel, tm_a, tm_b, tm_b_narrow, tm_xa, tm_xb, tm_xb_narrow, p) != cudaSuccess)
    return DICE_ERR_CUDA;
  return DICE_OK;
}
