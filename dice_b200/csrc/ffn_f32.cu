// fp32 expert FFN on the CUDA cores.
//
// The tensor cores round fp32 inputs to tf32, which cannot meet a 1e-5 parity
// bound, so the fp32 variant of the block runs this plain tiled kernel: 64x64
// output tile per CTA, 16-deep shared-memory slices, 4x4 register tile per
// thread, fmaf accumulation in ascending K.  Segments (experts) are ragged;
// each CTA finds its segment from the segment offsets on the device.
#include "common.cuh"

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

__device__ __forceinline__ float gelu_tanh_ref(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanhf(u));
}
__device__ __forceinline__ float silu_ref(float x) { return x / (1.0f + expf(-x)); }

template <int EPI>
__global__ void __launch_bounds__(256)
grouped_gemm_f32_kernel(const float* __restrict__ a, const float* __restrict__ w, const int* __restrict__ seg_offsets,
                        const int* __restrict__ seg_slab, int n_seg, int k_dim, int64_t w_rows, int n_out,
                        float* __restrict__ out, int64_t ld_out) {
  constexpr bool DUAL = EPI == DICE_EPI_SWIGLU;
  __shared__ int s_seg, s_row0, s_rows;
  __shared__ __align__(16) float As[TK][TM + 4];
  __shared__ __align__(16) float Ws[TK][TN + 4];
  __shared__ __align__(16) float Us[DUAL ? TK : 1][TN + 4];
  if (threadIdx.x == 0) {
    int run = 0, found = -1, row0 = 0, rows = 0;
    for (int s = 0; s < n_seg; ++s) {
      const int beg = seg_offsets[s], cnt = seg_offsets[s + 1] - beg;
      const int nb = cnt > 0 ? (cnt + TM - 1) / TM : 0;
      if (static_cast<int>(blockIdx.x) < run + nb) {
        found = s;
        row0 = beg + (blockIdx.x - run) * TM;
        rows = beg + cnt - row0;
        break;
      }
      run += nb;
    }
    s_seg = found; s_row0 = row0; s_rows = rows < TM ? rows : TM;
  }
  __syncthreads();
  if (s_seg < 0) return;
  const int slab = seg_slab != nullptr ? seg_slab[s_seg] : s_seg;
  if (slab < 0) return;  // rows that belong to no expert (the unused rest of a source's region)
  const float* wbase = w + static_cast<int64_t>(slab) * w_rows * k_dim;
  const int row0 = s_row0, rows = s_rows;
  const int col0 = blockIdx.y * TN;

  const int lr = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;  // loader: row lr, k offset lk
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  float acc[4][4], accu[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) { acc[i][j] = 0.f; accu[i][j] = 0.f; }

  // weight row feeding output column j
  const int j_glob = col0 + lr;
  int64_t wrow = -1, urow = -1;
  if (j_glob < n_out) {
    if (DUAL) {
      wrow = static_cast<int64_t>(j_glob / 128) * 256 + (j_glob % 128);
      urow = wrow + 128;
    } else {
      wrow = j_glob;
    }
  }

  for (int k0 = 0; k0 < k_dim; k0 += TK) {
    float4 av = make_float4(0.f, 0.f, 0.f, 0.f), wv = av, uv = av;
    const bool k_ok = k0 + lk < k_dim;  // k_dim % 4 == 0
    if (k_ok && lr < rows) av = *reinterpret_cast<const float4*>(a + static_cast<int64_t>(row0 + lr) * k_dim + k0 + lk);
    if (k_ok && wrow >= 0) wv = *reinterpret_cast<const float4*>(wbase + wrow * k_dim + k0 + lk);
    if (DUAL && k_ok && urow >= 0) uv = *reinterpret_cast<const float4*>(wbase + urow * k_dim + k0 + lk);
    As[lk + 0][lr] = av.x; As[lk + 1][lr] = av.y; As[lk + 2][lr] = av.z; As[lk + 3][lr] = av.w;
    Ws[lk + 0][lr] = wv.x; Ws[lk + 1][lr] = wv.y; Ws[lk + 2][lr] = wv.z; Ws[lk + 3][lr] = wv.w;
    if (DUAL) { Us[lk + 0][lr] = uv.x; Us[lk + 1][lr] = uv.y; Us[lk + 2][lr] = uv.z; Us[lk + 3][lr] = uv.w; }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      const float4 a4 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 b4 = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
      const float ar[4] = {a4.x, a4.y, a4.z, a4.w};
      const float br[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
      if (DUAL) {
        const float4 u4 = *reinterpret_cast<const float4*>(&Us[k][tx * 4]);
        const float ur[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) accu[i][j] = fmaf(ar[i], ur[j], accu[i][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx * 4 + j;
      if (c >= n_out) continue;
      float v = acc[i][j];
      if (EPI == DICE_EPI_GELU_TANH) v = gelu_tanh_ref(v);
      if (EPI == DICE_EPI_SWIGLU) v = silu_ref(v) * accu[i][j];
      out[static_cast<int64_t>(row0 + r) * ld_out + c] = v;
    }
  }
}

template <int EPI>
int launch_f32(const void* a, int64_t n_rows, int k_dim, const void* w, int64_t w_rows, const int32_t* seg_offsets,
               const int32_t* seg_slab, int n_seg, void* out, int64_t ld_out, int n_out, cudaStream_t s) {
  const int64_t gx = (n_rows + TM - 1) / TM + n_seg;
  const int gy = (n_out + TN - 1) / TN;
  if (gx > 0x7fffffffLL || gy > 65535) return DICE_ERR_LIMIT;
  dice_count_launch();
  grouped_gemm_f32_kernel<EPI><<<dim3(static_cast<unsigned>(gx), gy), 256, 0, s>>>(
      static_cast<const float*>(a), static_cast<const float*>(w), seg_offsets, seg_slab, n_seg, k_dim, w_rows, n_out,
      static_cast<float*>(out), ld_out);
  return cudaGetLastError() == cudaSuccess ? DICE_OK : DICE_ERR_CUDA;
}

}  // namespace

extern "C" int dice_grouped_ffn_f32(const void* rows_in, int64_t n_rows, int hidden, int ffn, int act, const void* w1,
                                    const void* w2, int n_slabs, const int32_t* seg_offsets, const int32_t* seg_slab,
                                    int n_seg, void* inter, void* rows_out, void* stream) {
  DICE_CHECK_ARG(act == DICE_ACT_SWIGLU || act == DICE_ACT_GELU_TANH, DICE_ERR_ARG);
  DICE_CHECK_ARG(n_rows >= 0 && hidden > 0 && ffn > 0 && n_slabs > 0 && n_seg >= 0, DICE_ERR_ARG);
  DICE_CHECK_ARG(hidden % 4 == 0 && ffn % 4 == 0, DICE_ERR_SHAPE);
  if (n_rows == 0 || n_seg == 0) return DICE_OK;
  DICE_CHECK_ARG(rows_in && w1 && w2 && seg_offsets && inter && rows_out, DICE_ERR_ARG);
  DICE_CHECK_ARG(dice_aligned16(rows_in) && dice_aligned16(w1) && dice_aligned16(w2) && dice_aligned16(inter),
                 DICE_ERR_ALIGN);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc;
  if (act == DICE_ACT_SWIGLU)
    rc = launch_f32<DICE_EPI_SWIGLU>(rows_in, n_rows, hidden, w1, dice_w13_rows(ffn), seg_offsets, seg_slab, n_seg,
                                     inter, ffn, ffn, s);
  else
    rc = launch_f32<DICE_EPI_GELU_TANH>(rows_in, n_rows, hidden, w1, ffn, seg_offsets, seg_slab, n_seg, inter, ffn, ffn,
                                        s);
  if (rc != DICE_OK) return rc;
  return launch_f32<DICE_EPI_STORE>(inter, n_rows, ffn, w2, hidden, seg_offsets, seg_slab, n_seg, rows_out, hidden,
                                    hidden, s);
}
