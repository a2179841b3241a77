// Shared helpers for the dice_b200 kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dice_b200.h"

#define DICE_CHECK_ARG(cond, code) \
  do {                             \
    if (!(cond)) return (code);    \
  } while (0)

#define DICE_CUDA_OK(expr)                         \
  do {                                             \
    if ((expr) != cudaSuccess) return DICE_ERR_CUDA; \
  } while (0)

// device status codes written by kernels whose bounded waits expired
#define DICE_STATUS_OK 0u
#define DICE_STATUS_WAIT_SMEM_FULL 1u   // tensor-core warp: operand tiles never arrived
#define DICE_STATUS_WAIT_SMEM_EMPTY 2u  // loader warp: ring slot never released
#define DICE_STATUS_WAIT_ACC_FULL 3u    // epilogue warps: accumulator never completed
#define DICE_STATUS_WAIT_ACC_EMPTY 4u   // tensor-core warp: accumulator never drained
#define DICE_STATUS_BAD_SEGMENTS 5u     // segment offsets not monotone / beyond n_rows
#define DICE_STATUS_WAIT_PEER_COUNTS 6u    // exchange: a peer's row counts never arrived
#define DICE_STATUS_WAIT_PEER_DISPATCH 7u  // exchange: a peer's dispatched rows never arrived
#define DICE_STATUS_WAIT_PEER_COMBINE 8u   // exchange: a peer's expert outputs never arrived
#define DICE_STATUS_EXCHANGE_OVERFLOW 9u   // exchange: more rows than the receive buffer holds
#define DICE_STATUS_PEER_FAILED 10u        // exchange: a source rank marked its push as incomplete
#define DICE_STATUS_WAIT_FFN_ROWS 11u      // exchange: the expert outputs a return push follows never completed

static inline bool dice_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static inline size_t dice_dtype_size(int dtype) {
  return dtype == DICE_BF16 ? 2 : (dtype == DICE_F32 ? 4 : 0);
}

// ---- programmatic dependent launch ------------------------------------------------
// Kernels started with dice_launch() may become resident while the kernel before them in the stream is still
// running (its blocks have all started and called pdl_trigger(), or exited).  Such a kernel does its set-up,
// then calls pdl_wait(), which returns once the earlier kernels have completed and their writes are visible;
// it touches no global memory before that.  Launch gaps and prologues then overlap the predecessor's tail.
// DICE_PDL=0 in the environment turns the launch attribute off (plain stream order).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool dice_pdl_enabled();  // abi.cu
void dice_count_launch();  // abi.cu: every kernel launch of the library is counted (dice_kernel_launches)

template <typename... KArgs, typename... Args>
static inline cudaError_t dice_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                      Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dice_pdl_enabled() ? 1 : 0;
  dice_count_launch();
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// plain stream order: the kernel starts only when everything before it in the stream has completed.  For a kernel
// behind work that shares the GPU with a kernel of another stream: blocks that became resident early would sit on
// the SMs left free for that other kernel.
template <typename... KArgs, typename... Args>
static inline cudaError_t dice_launch_ordered(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                              cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  dice_count_launch();
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// streaming 16-byte load (coherent: the kernels that use it may start while the producer of the data still runs)
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void stg_stream16(void* p, const uint4& v) {
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ float bf16lo_to_f32(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16hi_to_f32(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// internal (not exported): bf16 router on the tensor cores, defined next to the grouped GEMM kernel
int dice_internal_router_tc(const void* x, const void* w_gate, int64_t n_tokens, int hidden, int n_experts, int renorm,
                            int64_t* out_idx, float* out_w, int32_t* out_hist, int32_t* out_chunk_hist,
                            void* out_logits, uint32_t* status, cudaStream_t stream);

// internal (not exported): grouped GEMM on CTA pairs (cta_group::2); arguments as dice_grouped_gemm, validated by it
// where the output rows of a grouped GEMM go when they leave the GPU (see GemmParams::ret_*)
struct DiceReturnSpec {
  int world, rank, capacity_rows;
  const int32_t* meta;
  const void* const* bufs;   // host array [world]
  const void* const* flags;  // host array [world]
  uint32_t* done_counter;
  uint32_t seq;
};
// a dense problem (one segment, one weight slab) appended to the tile list of a grouped GEMM launch
struct DiceDenseSpec {
  const void* a;   // [n_rows, k_dim]
  int64_t n_rows;
  int k_dim;
  const void* w;   // [w_rows, k_dim]
  int64_t w_rows;
  void* out;       // [n_rows, ld_out]
  int64_t ld_out;
  int n_out;
};
// the weighted scatter-add of a grouped GEMM's rows into token rows (see dice_grouped_ffn_combine)
struct DiceCombineSpec {
  const int32_t* order;   // sorted position -> flat (token, slot) row
  const float* weights;   // gate weight of every flat row
};
int dice_internal_gemm_pair(const void* a, int64_t n_rows, int k_dim, const void* w, int n_slabs, int64_t w_rows,
                            const int32_t* seg_offsets, const int32_t* seg_slab, int n_seg, int epilogue, void* out,
                            int64_t ld_out, int n_out, int reserve_sms, uint32_t* status, cudaStream_t stream,
                            const DiceReturnSpec* ret = nullptr, const DiceDenseSpec* extra = nullptr,
                            const DiceCombineSpec* combine = nullptr, uint32_t* rows_done = nullptr);
// completions the CTA-pair kernel counts per 256-row block and output tile when rows_done is given
constexpr int kRowsDonePerTile = 16;  // 2 CTAs x 8 epilogue warps
