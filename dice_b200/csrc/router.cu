// Fused router: gate logits -> softmax -> top-2 -> expert histogram.
//
// One warp owns TOK consecutive tokens.  Each lane streams 16-byte chunks of
// the tokens' activation rows (read once from HBM, not kept in L1) and
// multiplies them with the matching chunks of every expert's gate row, which
// all warps of an SM share through L1.  Partial dot products are reduced with
// warp shuffles; one lane per token then rounds the logits to the activation
// type, selects the two largest and evaluates their softmax scores in fp32.
// HBM traffic is one pass over x plus a few bytes per token, so the kernel is
// bounded by HBM bandwidth.
#include <math.h>

#include "common.cuh"

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

// Top-2 of l[0..n_experts): larger first, lower index first among equals;
// softmax scores of the two in fp32.
template <int EP>
__device__ __forceinline__ void select_top2(const float (&l)[EP], int n_experts, int renorm, int& i0,
                                            int& i1, float& p0, float& p1) {
  float best0 = -INFINITY;
  i0 = 0;
#pragma unroll
  for (int e = 0; e < EP; ++e)
    if (e < n_experts && l[e] > best0) { best0 = l[e]; i0 = e; }
  float best1 = -INFINITY;
  i1 = (i0 == 0) ? 1 : 0;
#pragma unroll
  for (int e = 0; e < EP; ++e)
    if (e < n_experts && e != i0 && l[e] > best1) { best1 = l[e]; i1 = e; }
  float sum = 0.f;
#pragma unroll
  for (int e = 0; e < EP; ++e)
    if (e < n_experts) sum += expf(l[e] - best0);
  p0 = 1.0f / sum;
  p1 = expf(best1 - best0) / sum;
  if (renorm) {
    const float d = p0 + p1 + 1e-20f;
    p0 /= d;
    p1 /= d;
  }
}

__device__ __forceinline__ void write_choice(int64_t tok, int i0, int i1, float p0, float p1,
                                             int64_t* out_idx, float* out_w, int* s_hist) {
  longlong2 iv; iv.x = i0; iv.y = i1;
  *reinterpret_cast<longlong2*>(out_idx + 2 * tok) = iv;
  *reinterpret_cast<float2*>(out_w + 2 * tok) = make_float2(p0, p1);
  atomicAdd(&s_hist[i0], 1);
  atomicAdd(&s_hist[i1], 1);
}

template <typename T, int EP, int TOK>
__global__ void __launch_bounds__(kRouterWarps * 32)
router_top2_kernel(const T* __restrict__ x, const T* __restrict__ wg, int64_t n_tokens, int hidden,
                   int n_experts, int renorm, int64_t* __restrict__ out_idx, float* __restrict__ out_w,
                   int* __restrict__ hist, T* __restrict__ logits_out) {
  constexpr int EL = Chunk<T>::kElems;
  __shared__ int s_hist[EP];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x < EP) s_hist[threadIdx.x] = 0;
  __syncthreads();

  const int64_t tok0 = (static_cast<int64_t>(blockIdx.x) * kRouterWarps + warp) * TOK;
  const int n_chunks = hidden / EL;
  float acc[TOK][EP];
#pragma unroll
  for (int t = 0; t < TOK; ++t)
#pragma unroll
    for (int e = 0; e < EP; ++e) acc[t][e] = 0.f;

  if (tok0 < n_tokens) {
    for (int c = lane; c < n_chunks; c += 32) {
      float xv[TOK][EL];
#pragma unroll
      for (int t = 0; t < TOK; ++t) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (tok0 + t < n_tokens) v = ldg_stream16(x + (tok0 + t) * hidden + static_cast<int64_t>(c) * EL);
        Chunk<T>::unpack(v, xv[t]);
      }
#pragma unroll
      for (int e = 0; e < EP; ++e) {
        if (e < n_experts) {
          float wv[EL];
          Chunk<T>::unpack(__ldg(reinterpret_cast<const uint4*>(wg + static_cast<int64_t>(e) * hidden) + c), wv);
#pragma unroll
          for (int t = 0; t < TOK; ++t)
#pragma unroll
            for (int j = 0; j < EL; ++j) acc[t][e] = fmaf(xv[t][j], wv[j], acc[t][e]);
        }
      }
    }
#pragma unroll
    for (int t = 0; t < TOK; ++t)
#pragma unroll
      for (int e = 0; e < EP; ++e) {
        float v = acc[t][e];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        acc[t][e] = Chunk<T>::round_trip(v);
      }
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
      if (lane == t && tok0 + t < n_tokens) {
        const int64_t tok = tok0 + t;
        if (logits_out != nullptr) {
#pragma unroll
          for (int e = 0; e < EP; ++e)
            if (e < n_experts) Chunk<T>::store(logits_out + tok * n_experts + e, acc[t][e]);
        }
        int i0, i1; float p0, p1;
        select_top2<EP>(acc[t], n_experts, renorm, i0, i1, p0, p1);
        write_choice(tok, i0, i1, p0, p1, out_idx, out_w, s_hist);
      }
    }
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
  const int64_t tok_per_block = static_cast<int64_t>(kRouterWarps) * TOK;
  const int64_t blocks = (n + tok_per_block - 1) / tok_per_block;
  if (blocks > 0x7fffffffLL) return DICE_ERR_LIMIT;
  router_top2_kernel<T, EP, TOK><<<static_cast<unsigned>(blocks), kRouterWarps * 32, 0, s>>>(
      static_cast<const T*>(x), static_cast<const T*>(wg), n, h, e, renorm, idx, w, hist, static_cast<T*>(logits));
  return cudaGetLastError() == cudaSuccess ? DICE_OK : DICE_ERR_CUDA;
}

template <typename T>
int dispatch_router(const void* x, const void* wg, int64_t n, int h, int e, int renorm, int64_t* idx, float* w,
                    int32_t* hist, void* logits, cudaStream_t s) {
  if (e <= 8) return launch_router<T, 8, 4>(x, wg, n, h, e, renorm, idx, w, hist, logits, s);
  if (e <= 16) return launch_router<T, 16, 4>(x, wg, n, h, e, renorm, idx, w, hist, logits, s);
  if (e <= 32) return launch_router<T, 32, 2>(x, wg, n, h, e, renorm, idx, w, hist, logits, s);
  return launch_router<T, 64, 1>(x, wg, n, h, e, renorm, idx, w, hist, logits, s);
}

template <typename T, int EP>
int launch_select(const void* logits, int64_t n, int e, int renorm, int64_t* idx, float* w, int32_t* hist,
                  cudaStream_t s) {
  const int64_t blocks = (n + 127) / 128;
  if (blocks > 0x7fffffffLL) return DICE_ERR_LIMIT;
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
                                void* out_logits, void* stream) {
  DICE_CHECK_ARG(n_tokens >= 0 && hidden > 0, DICE_ERR_ARG);
  DICE_CHECK_ARG(n_experts >= 2 && n_experts <= 64, DICE_ERR_SHAPE);
  DICE_CHECK_ARG(dtype == DICE_BF16 || dtype == DICE_F32, DICE_ERR_DTYPE);
  DICE_CHECK_ARG((hidden * dice_dtype_size(dtype)) % 16 == 0, DICE_ERR_SHAPE);
  DICE_CHECK_ARG(out_hist != nullptr, DICE_ERR_ARG);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  DICE_CUDA_OK(cudaMemsetAsync(out_hist, 0, sizeof(int32_t) * n_experts, s));
  if (n_tokens == 0) return DICE_OK;
  DICE_CHECK_ARG(x && w_gate && out_idx && out_w, DICE_ERR_ARG);
  DICE_CHECK_ARG(dice_aligned16(x) && dice_aligned16(w_gate) && dice_aligned16(out_idx) &&
                     (reinterpret_cast<uintptr_t>(out_w) & 7u) == 0,
                 DICE_ERR_ALIGN);
  if (dtype == DICE_BF16)
    return dispatch_router<__nv_bfloat16>(x, w_gate, n_tokens, hidden, n_experts, renorm, out_idx, out_w, out_hist,
                                          out_logits, s);
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
