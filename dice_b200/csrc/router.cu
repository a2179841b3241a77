// Fused router: gate logits -> softmax -> top-2 -> expert histogram.
//
// Two kernels.  bf16 activations go to the tcgen05 kernel (grouped_gemm.cu): the
// logits are one 128 x E accumulator tile per 128 tokens and each epilogue
// thread selects for its own token.  fp32 activations must keep fp32 products,
// so they use the CUDA-core kernel below:
//
// Persistent CTAs stage slabs of consecutive token rows in shared memory with
// TMA bulk copies (double-buffered), so HBM requests stay queued while the
// previous slab is multiplied.  One warp owns TOK tokens of a slab: each lane
// takes 16-byte chunks of those rows and multiplies them with the matching
// chunks of every expert's gate row (shared by all warps of an SM through L1)
// using packed two-wide fp32 FMAs.  Partial dot products are reduced with warp
// shuffles; one lane per token then rounds the logits to the activation type,
// selects the two largest and evaluates their softmax scores in fp32.  HBM
// traffic is one pass over x plus a few bytes per token, so the kernel is
// bounded by HBM bandwidth.
#include <math.h>

#include "common.cuh"
#include "select.cuh"

namespace {

constexpr int kRouterWarps = 4;

template <typename T>
struct Chunk;  // a 16-byte chunk of T as floats

template <>
struct Chunk<__nv_bfloat16> {
  static constexpr int kElems = 8;
  __device__ static void unpack(const uint4& v, float* f) {
    f[0] = bf16lo_to_f32(v.x); f[1] = bf16hi_to_f32(v.x);
    f[2] = bf16lo_to_f32(v.y); f[3] = bf16hi_to_f32(v.y);
    f[4] = bf16lo_to_f32(v.z); f[5] = bf16hi_to_f32(v.z);
    f[6] = bf16lo_to_f32(v.w); f[7] = bf16hi_to_f32(v.w);
  }
  __device__ static float round_trip(float a) { return __bfloat162float(__float2bfloat16_rn(a)); }
  __device__ static float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  __device__ static void store(__nv_bfloat16* p, float a) { *p = __float2bfloat16_rn(a); }
};

template <>
struct Chunk<float> {
  static constexpr int kElems = 4;
  __device__ static void unpack(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
  __device__ static float round_trip(float a) { return a; }
  __device__ static float load(const float* p) { return *p; }
  __device__ static void store(float* p, float a) { *p = a; }
};

__device__ __forceinline__ void write_choice(int64_t tok, int i0, int i1, float p0, float p1,
                                             int64_t* out_idx, float* out_w, int* s_hist) {
  longlong2 iv; iv.x = i0; iv.y = i1;
  *reinterpret_cast<longlong2*>(out_idx + 2 * tok) = iv;
  *reinterpret_cast<float2*>(out_w + 2 * tok) = make_float2(p0, p1);
  atomicAdd(&s_hist[i0], 1);
  atomicAdd(&s_hist[i1], 1);
}

// ---- bulk-copy helpers (TMA 1-D copies completing on an mbarrier) ---------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_try_wait(uint32_t bar, uint32_t parity) {
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
// bounded: a copy that has not landed after ~2^22 polls (seconds) is given up
__device__ __forceinline__ bool bar_wait_bounded(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < (1u << 22); ++i)
    if (bar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// Persistent CTAs of 4 warps walk tiles of 4*TOK consecutive tokens.  A tile is one
// contiguous slab of x, brought into shared memory by a single bulk copy; two slabs are
// in flight per CTA (the next tile loads while this one is multiplied), several CTAs
// share an SM, so HBM always has requests queued.
template <typename T, int EP, int TOK>
__global__ void __launch_bounds__(kRouterWarps * 32)
router_top2_kernel(const T* __restrict__ x, const T* __restrict__ wg, int64_t n_tokens, int hidden,
                   int n_experts, int renorm, int64_t* __restrict__ out_idx, float* __restrict__ out_w,
                   int* __restrict__ hist, T* __restrict__ logits_out) {
  constexpr int EL = Chunk<T>::kElems;
  constexpr int TOKB = kRouterWarps * TOK;
  extern __shared__ __align__(128) uint8_t slab[];
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ int s_hist[EP];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t row_bytes = static_cast<uint32_t>(hidden) * sizeof(T);
  const uint32_t tile_bytes = TOKB * row_bytes;
  const int64_t n_tiles = (n_tokens + TOKB - 1) / TOKB;
  const uint32_t bar0 = smem_addr(&bars[0]);

  if (threadIdx.x == 0) {
    bar_init(bar0, 1);
    bar_init(bar0 + 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < EP) s_hist[threadIdx.x] = 0;
  __syncthreads();

  auto issue = [&](int64_t tile, int stage) {
    const int64_t tok0 = tile * TOKB;
    const int64_t left = n_tokens - tok0;
    const uint32_t bytes = (left < TOKB ? static_cast<uint32_t>(left) : TOKB) * row_bytes;
    bar_expect_tx(bar0 + 8 * stage, bytes);
    bulk_load(smem_addr(slab) + stage * tile_bytes, x + tok0 * hidden, bytes, bar0 + 8 * stage);
  };

  int64_t tile = blockIdx.x;
  if (threadIdx.x == 0 && tile < n_tiles) issue(tile, 0);
  const int n_chunks = hidden / EL;
  for (int it = 0; tile < n_tiles; tile += gridDim.x, ++it) {
    const int stage = it & 1;
    if (threadIdx.x == 0 && tile + gridDim.x < n_tiles) issue(tile + gridDim.x, stage ^ 1);
    const bool landed = bar_wait_bounded(bar0 + 8 * stage, (it >> 1) & 1);
    const int64_t tok0 = tile * TOKB + warp * TOK;
    if (__syncthreads_or(!landed)) {
      // the copy never arrived: mark the tile's tokens as unrouted (expert -1, weight 0) and stop
      if (lane < TOK && tok0 + lane < n_tokens) {
        longlong2 iv; iv.x = -1; iv.y = -1;
        *reinterpret_cast<longlong2*>(out_idx + 2 * (tok0 + lane)) = iv;
        *reinterpret_cast<float2*>(out_w + 2 * (tok0 + lane)) = make_float2(0.f, 0.f);
      }
      break;
    }
    const uint4* xs = reinterpret_cast<const uint4*>(slab + stage * tile_bytes + static_cast<uint32_t>(warp * TOK) * row_bytes);
    const int row_vec = n_chunks;  // 16-byte chunks per row
    float2 acc[TOK][EP / 2];
#pragma unroll
    for (int t = 0; t < TOK; ++t)
#pragma unroll
      for (int e = 0; e < EP / 2; ++e) acc[t][e] = make_float2(0.f, 0.f);

    if (tok0 < n_tokens) {
      for (int c = lane; c < n_chunks; c += 32) {
        float xv[TOK][EL];
#pragma unroll
        for (int t = 0; t < TOK; ++t) Chunk<T>::unpack(xs[t * row_vec + c], xv[t]);
#pragma unroll
        for (int e = 0; e < EP; e += 2) {
          if (e < n_experts) {
            float w0[EL], w1[EL];
            Chunk<T>::unpack(__ldg(reinterpret_cast<const uint4*>(wg + static_cast<int64_t>(e) * hidden) + c), w0);
            if (e + 1 < n_experts) {
              Chunk<T>::unpack(__ldg(reinterpret_cast<const uint4*>(wg + static_cast<int64_t>(e + 1) * hidden) + c), w1);
            } else {
#pragma unroll
              for (int j = 0; j < EL; ++j) w1[j] = 0.f;
            }
#pragma unroll
            for (int t = 0; t < TOK; ++t)
#pragma unroll
              for (int j = 0; j < EL; ++j)
                acc[t][e / 2] = __ffma2_rn(make_float2(xv[t][j], xv[t][j]), make_float2(w0[j], w1[j]), acc[t][e / 2]);
          }
        }
      }
      float logit[TOK][EP];
#pragma unroll
      for (int t = 0; t < TOK; ++t)
#pragma unroll
        for (int e = 0; e < EP; ++e) {
          float v = (e & 1) ? acc[t][e / 2].y : acc[t][e / 2].x;
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
          logit[t][e] = Chunk<T>::round_trip(v);
        }
#pragma unroll
      for (int t = 0; t < TOK; ++t) {
        if (lane == t && tok0 + t < n_tokens) {
          const int64_t tok = tok0 + t;
          if (logits_out != nullptr) {
#pragma unroll
            for (int e = 0; e < EP; ++e)
              if (e < n_experts) Chunk<T>::store(logits_out + tok * n_experts + e, logit[t][e]);
          }
          int i0, i1; float p0, p1;
          select_top2<EP>(logit[t], n_experts, renorm, i0, i1, p0, p1);
          write_choice(tok, i0, i1, p0, p1, out_idx, out_w, s_hist);
        }
      }
    }
    __syncthreads();  // every warp is done with this slab before the next copy overwrites it
  }
  __syncthreads();
  if (threadIdx.x < n_experts && s_hist[threadIdx.x] != 0) atomicAdd(&hist[threadIdx.x], s_hist[threadIdx.x]);
}

template <typename T, int EP>
__global__ void __launch_bounds__(128)
top2_from_logits_kernel(const T* __restrict__ logits, int64_t n_tokens, int n_experts, int renorm,
                        int64_t* __restrict__ out_idx, float* __restrict__ out_w, int* __restrict__ hist) {
  __shared__ int s_hist[EP];
  if (threadIdx.x < EP) s_hist[threadIdx.x] = 0;
  __syncthreads();
  const int64_t tok = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tok < n_tokens) {
    float l[EP];
#pragma unroll
    for (int e = 0; e < EP; ++e) l[e] = (e < n_experts) ? Chunk<T>::load(logits + tok * n_experts + e) : 0.f;
    int i0, i1; float p0, p1;
    select_top2<EP>(l, n_experts, renorm, i0, i1, p0, p1);
    write_choice(tok, i0, i1, p0, p1, out_idx, out_w, s_hist);
  }
  __syncthreads();
  if (threadIdx.x < n_experts && s_hist[threadIdx.x] != 0) atomicAdd(&hist[threadIdx.x], s_hist[threadIdx.x]);
}

template <typename T, int EP, int TOK>
int launch_router(const void* x, const void* wg, int64_t n, int h, int e, int renorm, int64_t* idx, float* w,
                  int32_t* hist, void* logits, cudaStream_t s) {
  constexpr int TOKB = kRouterWarps * TOK;
  const size_t smem = 2 * static_cast<size_t>(TOKB) * h * sizeof(T);
  auto kernel = router_top2_kernel<T, EP, TOK>;
  static bool configured[64] = {false};
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return DICE_ERR_CUDA;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return DICE_ERR_CUDA;
  if (smem > 200 * 1024) return DICE_ERR_LIMIT;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
      return DICE_ERR_CUDA;
    configured[dev] = true;
  }
  const int64_t n_tiles = (n + TOKB - 1) / TOKB;
  int per_sm = static_cast<int>((220 * 1024) / (smem + 1024));
  per_sm = per_sm < 1 ? 1 : (per_sm > 6 ? 6 : per_sm);
  const int64_t grid = n_tiles < static_cast<int64_t>(sms) * per_sm ? n_tiles : static_cast<int64_t>(sms) * per_sm;
  dice_count_launch();
  kernel<<<static_cast<unsigned>(grid), kRouterWarps * 32, smem, s>>>(static_cast<const T*>(x), static_cast<const T*>(wg),
                                                                      n, h, e, renorm, idx, w, hist,
                                                                      static_cast<T*>(logits));
  return cudaGetLastError() == cudaSuccess ? DICE_OK : DICE_ERR_CUDA;
}

// tokens per warp chosen so that one slab (4 warps) stays near 36 KB
template <typename T, int EP>
int dispatch_tok(const void* x, const void* wg, int64_t n, int h, int e, int renorm, int64_t* idx, float* w,
                 int32_t* hist, void* logits, cudaStream_t s) {
  const size_t row = static_cast<size_t>(h) * sizeof(T);
  if (EP <= 16 && row * 16 <= 40 * 1024) return launch_router<T, EP, 4>(x, wg, n, h, e, renorm, idx, w, hist, logits, s);
  if (EP <= 32 && row * 8 <= 40 * 1024) return launch_router<T, EP, 2>(x, wg, n, h, e, renorm, idx, w, hist, logits, s);
  return launch_router<T, EP, 1>(x, wg, n, h, e, renorm, idx, w, hist, logits, s);
}

template <typename T>
int dispatch_router(const void* x, const void* wg, int64_t n, int h, int e, int renorm, int64_t* idx, float* w,
                    int32_t* hist, void* logits, cudaStream_t s) {
  if (e <= 8) return dispatch_tok<T, 8>(x, wg, n, h, e, renorm, idx, w, hist, logits, s);
  if (e <= 16) return dispatch_tok<T, 16>(x, wg, n, h, e, renorm, idx, w, hist, logits, s);
  if (e <= 32) return dispatch_tok<T, 32>(x, wg, n, h, e, renorm, idx, w, hist, logits, s);
  return dispatch_tok<T, 64>(x, wg, n, h, e, renorm, idx, w, hist, logits, s);
}

template <typename T, int EP>
int launch_select(const void* logits, int64_t n, int e, int renorm, int64_t* idx, float* w, int32_t* hist,
                  cudaStream_t s) {
  const int64_t blocks = (n + 127) / 128;
  if (blocks > 0x7fffffffLL) return DICE_ERR_LIMIT;
  dice_count_launch();
  top2_from_logits_kernel<T, EP><<<static_cast<unsigned>(blocks), 128, 0, s>>>(static_cast<const T*>(logits), n, e,
                                                                              renorm, idx, w, hist);
  return cudaGetLastError() == cudaSuccess ? DICE_OK : DICE_ERR_CUDA;
}

template <typename T>
int dispatch_select(const void* logits, int64_t n, int e, int renorm, int64_t* idx, float* w, int32_t* hist,
                    cudaStream_t s) {
  if (e <= 8) return launch_select<T, 8>(logits, n, e, renorm, idx, w, hist, s);
  if (e <= 16) return launch_select<T, 16>(logits, n, e, renorm, idx, w, hist, s);
  if (e <= 32) return launch_select<T, 32>(logits, n, e, renorm, idx, w, hist, s);
  return launch_select<T, 64>(logits, n, e, renorm, idx, w, hist, s);
}

}  // namespace

extern "C" int dice_router_top2(const void* x, const void* w_gate, int64_t n_tokens, int hidden, int n_experts,
                                int dtype, int renorm, int64_t* out_idx, float* out_w, int32_t* out_hist,
                                int32_t* out_chunk_hist, void* out_logits, uint32_t* status, void* stream) {
  DICE_CHECK_ARG(n_tokens >= 0 && hidden > 0, DICE_ERR_ARG);
  DICE_CHECK_ARG(n_experts >= 2 && n_experts <= 64, DICE_ERR_SHAPE);
  DICE_CHECK_ARG(dtype == DICE_BF16 || dtype == DICE_F32, DICE_ERR_DTYPE);
  DICE_CHECK_ARG((hidden * dice_dtype_size(dtype)) % 16 == 0, DICE_ERR_SHAPE);
  // per-chunk histograms come out of the tensor-core kernel's 128-token tiles; the fp32 kernel walks smaller tiles
  DICE_CHECK_ARG(out_chunk_hist == nullptr || dtype == DICE_BF16, DICE_ERR_DTYPE);
  DICE_CHECK_ARG(out_hist != nullptr || out_chunk_hist != nullptr, DICE_ERR_ARG);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out_hist != nullptr) DICE_CUDA_OK(cudaMemsetAsync(out_hist, 0, sizeof(int32_t) * n_experts, s));
  if (n_tokens == 0) return DICE_OK;
  DICE_CHECK_ARG(x && w_gate && out_idx && out_w, DICE_ERR_ARG);
  DICE_CHECK_ARG(dice_aligned16(x) && dice_aligned16(w_gate) && dice_aligned16(out_idx) &&
                     (reinterpret_cast<uintptr_t>(out_w) & 7u) == 0,
                 DICE_ERR_ALIGN);
  // bf16: the logits are a skinny GEMM on the tensor cores with the selection in its epilogue;
  // fp32 must not be rounded to tf32, so it takes the CUDA-core kernel of this file
  if (dtype == DICE_BF16)
    return dice_internal_router_tc(x, w_gate, n_tokens, hidden, n_experts, renorm, out_idx, out_w, out_hist,
                                   out_chunk_hist, out_logits, status, s);
  return dispatch_router<float>(x, w_gate, n_tokens, hidden, n_experts, renorm, out_idx, out_w, out_hist, out_logits,
                                s);
}

extern "C" int dice_top2_from_logits(const void* logits, int64_t n_tokens, int n_experts, int dtype, int renorm,
                                     int64_t* out_idx, float* out_w, int32_t* out_hist, void* stream) {
  DICE_CHECK_ARG(n_tokens >= 0, DICE_ERR_ARG);
  DICE_CHECK_ARG(n_experts >= 2 && n_experts <= 64, DICE_ERR_SHAPE);
  DICE_CHECK_ARG(dtype == DICE_BF16 || dtype == DICE_F32, DICE_ERR_DTYPE);
  DICE_CHECK_ARG(out_hist != nullptr, DICE_ERR_ARG);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  DICE_CUDA_OK(cudaMemsetAsync(out_hist, 0, sizeof(int32_t) * n_experts, s));
  if (n_tokens == 0) return DICE_OK;
  DICE_CHECK_ARG(logits && out_idx && out_w, DICE_ERR_ARG);
  DICE_CHECK_ARG(dice_aligned16(out_idx) && (reinterpret_cast<uintptr_t>(out_w) & 7u) == 0, DICE_ERR_ALIGN);
  if (dtype == DICE_BF16)
    return dispatch_select<__nv_bfloat16>(logits, n_tokens, n_experts, renorm, out_idx, out_w, out_hist, s);
  return dispatch_select<float>(logits, n_tokens, n_experts, renorm, out_idx, out_w, out_hist, s);
}
