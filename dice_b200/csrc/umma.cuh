// tcgen05 / TMA / mbarrier building blocks shared by the tensor-core kernels
// (grouped_gemm.cu: one CTA per tile; grouped_gemm_pair.cu: CTA pairs).
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace dice_umma {

constexpr int BM = 128;          // rows per tile (tensor-memory lanes)
constexpr int BN = 256;          // weight rows per tile (accumulator columns)
constexpr int BK = 64;           // reduction elements per ring slot (128 bytes of bf16)
constexpr int UMMA_K = 16;       // reduction elements per tcgen05.mma
constexpr int kStages = 4;      // ring slots when the weight box is full-size (48 KB per slot)
constexpr int kMaxStages = 10;  // ring slots when the weight box is small (router: 18 KB per slot)
constexpr int kAccStages = 2;
constexpr int kTileABytes = BM * BK * 2;
constexpr int kTileBBytes = BN * BK * 2;
constexpr int kStageBytes = kTileABytes + kTileBBytes;
constexpr int kThreads = 320;       // warp 0 loader, warp 1 tensor-core issue, warps 2..9 epilogue
constexpr int kEpilogueWarps = 8;   // two per tensor-memory lane quadrant, alternating 32-column chunks
constexpr int kMaxSeg = 256;
constexpr int kTmemCols = 512;
constexpr uint64_t kWaitLimitNs = 1000ull * 1000ull * 1000ull;  // 1 s per wait
constexpr int kAuxBytes = 4096;  // barriers, flags and the segment tables
constexpr int kSmemBytes = kStages * kStageBytes + kAuxBytes + 1024;  // +1024: manual alignment

constexpr int kMaxPeerRanks = 16;

struct GemmParams {
  const int* seg_offsets;
  const int* seg_slab;
  int n_seg;
  int n_rows;
  int n_kblk;      // ceil(k_dim / BK)
  int n_nblk;      // ceil(w_rows / BN)
  int w_rows;      // weight rows per slab
  int n_out;       // logical output columns
  int epilogue;
  __nv_bfloat16* out;
  int64_t ld_out;
  uint32_t* status;
  int b_box_rows;  // rows of the weight box one TMA load brings (<= BN)
  int n_stages;    // ring depth: as many slots as fit, between kStages and kMaxStages
  // router epilogue only
  int n_experts;
  int renorm;
  int64_t* out_idx;
  float* out_w;
  int* hist;        // [n_experts] totals (may be null)
  int* chunk_hist;  // [tiles][n_experts] per-128-token histograms (may be null)
  __nv_bfloat16* logits_out;
  // A second, dense problem (one segment, one weight slab) whose tiles follow the first problem's in the tile list
  // of the same launch (CTA-pair kernel only; x_rows == 0: none).  It has its own operands (separate tensor maps)
  // and its own reduction depth and output; the epilogue kind is the launch's.
  int x_rows, x_kblk, x_nblk, x_w_rows, x_n_out;
  __nv_bfloat16* x_out;
  int64_t x_ld_out;
  // when set (CTA-pair kernel, first problem only): every epilogue warp adds 1 to rows_done[m-block] after its
  // stores of a tile are visible, so that a concurrent kernel can follow the output block by block
  unsigned int* rows_done;
#ifdef DICE_FOLLOW_TRACE
  int trace_id;
#endif
  // combine epilogue (CTA-pair kernel only): sorted position -> flat (token, slot) row, and the flat rows' gate weights
  const int* cmb_order;
  const float* cmb_weights;
  // output rows leave the GPU (CTA-pair kernel only): row r of the receive order belongs to source rank s
  // with ret_src_off[s] <= r < ret_src_off[s+1] and is stored in that rank's buffer at row
  // ret_back_base[s] + r - ret_src_off[s]; ret_world == 0 means a plain local store to `out`
  int ret_world;
  int ret_rank;
  int ret_capacity_rows;
  const int* ret_meta;            // meta block of the exchange (p2p_exchange.cu)
  void* ret_bufs[kMaxPeerRanks];  // peers' combine buffers
  uint32_t* ret_flags[kMaxPeerRanks];
  unsigned int* ret_done_counter;
  uint32_t ret_seq;
};

constexpr int kEpiRouter = 100;   // internal epilogue: logits -> top-2 (see launch_router_tc)
constexpr int kEpiCombine = 101;  // internal epilogue (CTA-pair kernel): out[token(r)] += weight(r) * row r

// ---- PTX wrappers ---------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Wait for `parity` of `bar`; give up after kWaitLimitNs or when another role
// has already given up.  Returns false when the caller must leave its loop.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                            uint32_t* status, uint32_t code) {
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 127u) == 0) {
      if (*abort_flag != 0) return false;
      if (global_timer_ns() - t0 > kWaitLimitNs) {
        if (status != nullptr) atomicCAS(status, 0u, code);
        *abort_flag = 1;
        __threadfence_block();
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          uint32_t* status, uint32_t code) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, status, code);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}

// One lane of a converged warp.  Producer loops run warp-wide and elect a lane for the TMA / MMA
// instructions, which keeps their loop state warp-uniform for the compiler.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem_addr, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem_addr), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// Shared-memory operand descriptor: K-major tile of 128-byte rows written by
// TMA with the 128-byte swizzle; 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t make_operand_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);  // start address / 16
  d |= static_cast<uint64_t>(1) << 16;                        // leading byte offset (unused with swizzle)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                // stride byte offset: 8 rows * 128 B
  d |= static_cast<uint64_t>(1) << 46;                        // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                        // 128-byte swizzle
  return d;
}

// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major.
__device__ __forceinline__ uint32_t make_instr_desc(int m, int n) {
  uint32_t d = 0;
  d |= 1u << 4;                              // accumulator format: fp32
  d |= 1u << 7;                              // A format: bf16
  d |= 1u << 10;                             // B format: bf16
  d |= static_cast<uint32_t>(n >> 3) << 17;  // N / 8
  d |= static_cast<uint32_t>(m >> 4) << 24;  // M / 16
  return d;
}

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float u = 0.7978845608028654f * fmaf(0.044715f * x * x, x, x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.0f + t);
}
__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// Store 32 consecutive output columns of one row; columns at or beyond
// `n_valid` (relative to the first of the 32) are dropped in groups of 8.
__device__ __forceinline__ void store_row_chunk(__nv_bfloat16* dst, const float (&v)[32], int n_valid, bool row_ok) {
  if (!row_ok) return;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    if (g * 8 < n_valid) {
      uint4 o = make_uint4(pack_bf16x2(v[g * 8 + 0], v[g * 8 + 1]), pack_bf16x2(v[g * 8 + 2], v[g * 8 + 3]),
                           pack_bf16x2(v[g * 8 + 4], v[g * 8 + 5]), pack_bf16x2(v[g * 8 + 6], v[g * 8 + 7]));
      *reinterpret_cast<uint4*>(dst + g * 8) = o;
    }
  }
}


// ---- host side, shared ------------------------------------------------------------
int encode_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);
int sm_count_cached();

}  // namespace dice_umma
