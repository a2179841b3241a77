// The element-wise work of the DiT block around the MoE block, one pass each:
//
//   x_in = LayerNorm(x) * (1 + scale[b]) + shift[b]        (in front of the router / the row gather)
//
// where b is the sample a token belongs to and the LayerNorm has no affine
// parameters.  PyTorch runs this as a normalisation kernel plus two or three
// element-wise kernels, each a full pass over [N, h]; here every activation
// byte is read once and written once.  (The other half of the glue, the gated
// residual `x + gate[b] * y`, is part of the combine kernel in permute.cu.)
//
// One warp owns a token: the row lives in registers between the two reduction
// passes (mean, then the sum of squared deviations, both in fp32), so the
// kernel is bounded by HBM bandwidth.
#include "common.cuh"

namespace {

constexpr int kMaxRowElems = 2048;  // a lane holds 64 values of its token's row

template <typename T>
struct Elem;
template <>
struct Elem<__nv_bfloat16> {
  static constexpr int kPerChunk = 8;
  __device__ static void unpack(const uint4& v, float* f) {
    f[0] = bf16lo_to_f32(v.x); f[1] = bf16hi_to_f32(v.x); f[2] = bf16lo_to_f32(v.y); f[3] = bf16hi_to_f32(v.y);
    f[4] = bf16lo_to_f32(v.z); f[5] = bf16hi_to_f32(v.z); f[6] = bf16lo_to_f32(v.w); f[7] = bf16hi_to_f32(v.w);
  }
};
template <>
struct Elem<float> {
  static constexpr int kPerChunk = 4;
  __device__ static void unpack(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
};

// stores `n` consecutive floats as TOut, 16 bytes at a time
__device__ __forceinline__ void store_chunk(__nv_bfloat16* dst, const float* f) {
  *reinterpret_cast<uint4*>(dst) =
      make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}
__device__ __forceinline__ void store_chunk(float* dst, const float* f) {
  *reinterpret_cast<float4*>(dst) = make_float4(f[0], f[1], f[2], f[3]);
}

// MAXC: 16-byte chunks of the row one lane holds (the row stays in registers in its storage format and is
// unpacked in each pass, so a bf16 row of 1152 costs 20 registers per lane and several CTAs share an SM)
template <typename TIn, typename TOut, int MAXC>
__global__ void __launch_bounds__(256)
ln_modulate_kernel(const TIn* __restrict__ x, const TIn* __restrict__ shift, const TIn* __restrict__ scale,
                   int64_t n_tokens, int hidden, int tokens_per_sample, float eps, TOut* __restrict__ out) {
  constexpr int EL = Elem<TIn>::kPerChunk;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * 8 + warp;
  pdl_trigger();
  pdl_wait();
  if (t >= n_tokens) return;
  const int n_chunks = hidden / EL;
  const uint4* row = reinterpret_cast<const uint4*>(x + t * hidden);
  uint4 raw[MAXC];
#pragma unroll
  for (int i = 0; i < MAXC; ++i)
    if (lane + 32 * i < n_chunks) raw[i] = ldg_stream16(row + lane + 32 * i);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    if (lane + 32 * i < n_chunks) {
      float v[EL];
      Elem<TIn>::unpack(raw[i], v);
#pragma unroll
      for (int j = 0; j < EL; ++j) sum += v[j];
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  const float mean = sum / static_cast<float>(hidden);
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    if (lane + 32 * i < n_chunks) {
      float v[EL];
      Elem<TIn>::unpack(raw[i], v);
#pragma unroll
      for (int j = 0; j < EL; ++j) {
        const float d = v[j] - mean;
        sq = fmaf(d, d, sq);
      }
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
  const float rstd = rsqrtf(sq / static_cast<float>(hidden) + eps);
  const int64_t b = t / tokens_per_sample;
  const uint4* sh = reinterpret_cast<const uint4*>(shift + b * hidden);
  const uint4* sc = reinterpret_cast<const uint4*>(scale + b * hidden);
  TOut* o = out + t * hidden;
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    const int c = lane + 32 * i;
    if (c < n_chunks) {
      float v[EL], s[EL], m[EL], r[EL];
      Elem<TIn>::unpack(raw[i], v);
      Elem<TIn>::unpack(__ldg(sh + c), s);
      Elem<TIn>::unpack(__ldg(sc + c), m);
#pragma unroll
      for (int j = 0; j < EL; ++j) r[j] = fmaf((v[j] - mean) * rstd, 1.f + m[j], s[j]);
      if constexpr (EL == 8 && sizeof(TOut) == 2) {
        store_chunk(reinterpret_cast<__nv_bfloat16*>(o) + c * 8, r);
      } else if constexpr (EL == 4 && sizeof(TOut) == 4) {
        store_chunk(reinterpret_cast<float*>(o) + c * 4, r);
      } else {
        // mixed widths (fp32 in, bf16 out): 4 values = 8 bytes
#pragma unroll
        for (int j = 0; j < EL; j += 2)
          *reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(o) + c * EL + j) = pack_bf16x2(r[j], r[j + 1]);
      }
    }
  }
}

template <typename TIn, typename TOut, int MAXC>
cudaError_t launch_ln(const void* x, const void* shift, const void* scale, int64_t n_tokens, int hidden, int tps, float eps,
                      void* out, cudaStream_t s) {
  const dim3 grid(static_cast<unsigned>((n_tokens + 7) / 8));
  return dice_launch(ln_modulate_kernel<TIn, TOut, MAXC>, grid, dim3(256), 0, s, static_cast<const TIn*>(x),
                     static_cast<const TIn*>(shift), static_cast<const TIn*>(scale), n_tokens, hidden, tps, eps,
                     static_cast<TOut*>(out));
}

// the smallest instantiation whose lanes can hold the row
template <typename TIn, typename TOut>
cudaError_t dispatch_ln(const void* x, const void* shift, const void* scale, int64_t n_tokens, int hidden, int tps, float eps,
                        void* out, cudaStream_t s) {
  constexpr int EL = Elem<TIn>::kPerChunk;
  constexpr int kFull = kMaxRowElems / 32 / EL;  // 8 (bf16) or 16 (fp32) chunks per lane
  const int per_lane = (hidden / EL + 31) / 32;
  if (per_lane <= kFull / 4) return launch_ln<TIn, TOut, kFull / 4>(x, shift, scale, n_tokens, hidden, tps, eps, out, s);
  if (per_lane <= (kFull * 5) / 8) return launch_ln<TIn, TOut, (kFull * 5) / 8>(x, shift, scale, n_tokens, hidden, tps, eps, out, s);
  return launch_ln<TIn, TOut, kFull>(x, shift, scale, n_tokens, hidden, tps, eps, out, s);
}

}  // namespace

extern "C" int dice_ln_modulate(const void* x, const void* shift, const void* scale, int64_t n_tokens, int hidden,
                                int tokens_per_sample, float eps, int dtype, int out_dtype, void* out, void* stream) {
  DICE_CHECK_ARG(n_tokens >= 0 && hidden > 0 && tokens_per_sample > 0 && eps >= 0.f, DICE_ERR_ARG);
  const size_t es = dice_dtype_size(dtype), os = dice_dtype_size(out_dtype);
  DICE_CHECK_ARG(es != 0 && os != 0, DICE_ERR_DTYPE);
  DICE_CHECK_ARG(!(dtype == DICE_BF16 && out_dtype == DICE_F32), DICE_ERR_DTYPE);  // no widening form
  DICE_CHECK_ARG((hidden * es) % 16 == 0 && (hidden * os) % 16 == 0, DICE_ERR_SHAPE);
  DICE_CHECK_ARG(hidden <= kMaxRowElems, DICE_ERR_LIMIT);
  if (n_tokens == 0) return DICE_OK;
  DICE_CHECK_ARG(x && shift && scale && out, DICE_ERR_ARG);
  DICE_CHECK_ARG(dice_aligned16(x) && dice_aligned16(shift) && dice_aligned16(scale) && dice_aligned16(out), DICE_ERR_ALIGN);
  const int64_t blocks = (n_tokens + 7) / 8;
  DICE_CHECK_ARG(blocks <= 0x7fffffffLL, DICE_ERR_LIMIT);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err;
  if (dtype == DICE_BF16)
    err = dispatch_ln<__nv_bfloat16, __nv_bfloat16>(x, shift, scale, n_tokens, hidden, tokens_per_sample, eps, out, s);
  else if (out_dtype == DICE_F32)
    err = dispatch_ln<float, float>(x, shift, scale, n_tokens, hidden, tokens_per_sample, eps, out, s);
  else
    err = dispatch_ln<float, __nv_bfloat16>(x, shift, scale, n_tokens, hidden, tokens_per_sample, eps, out, s);
  return err == cudaSuccess ? DICE_OK : DICE_ERR_CUDA;
}
