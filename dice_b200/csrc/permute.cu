// Token permutation for the MoE block: a stable counting sort of the
// (token, slot) rows by expert, the 128-bit row gather into expert-sorted
// order, and the inverse gather fused with the gate-weighted pair sum.
//
// The plan works on 4-byte indices only (a few hundred KB); the two row movers
// read and write every activation byte exactly once and are bounded by HBM
// bandwidth.
#include <mutex>

#include "common.cuh"

// Scratch of dice_permute_plan_static: lives in the library image, so every GPU that loads the
// library holds these 256 KB until the process exits.  Host code may only use this name to ask
// for the array's device address (cudaGetSymbolAddress); it is not itself a device pointer.
static __device__ __align__(256) int g_plan_static_scratch[DICE_PLAN_STATIC_MAX_INTS];

namespace {

constexpr int kChunkRows = 256;  // rows ranked by one thread block
constexpr int kMaxExperts = 64;

// ---- plan, pass 1: per-chunk expert histogram -------------------------------
__global__ void __launch_bounds__(kChunkRows)
plan_count_kernel(const int64_t* __restrict__ flat_idx, int64_t n_rows, int n_experts, int* __restrict__ chunk_hist) {
  __shared__ int s_hist[kMaxExperts];
  pdl_trigger();
  if (threadIdx.x < kMaxExperts) s_hist[threadIdx.x] = 0;
  __syncthreads();
  pdl_wait();
  const int64_t r = static_cast<int64_t>(blockIdx.x) * kChunkRows + threadIdx.x;
  if (r < n_rows) {
    const int64_t e = flat_idx[r];
    if (e >= 0 && e < n_experts) atomicAdd(&s_hist[e], 1);
  }
  __syncthreads();
  if (threadIdx.x < n_experts) chunk_hist[static_cast<int64_t>(blockIdx.x) * n_experts + threadIdx.x] = s_hist[threadIdx.x];
}

// ---- plan, pass 2: exclusive scan over chunks (per expert) and experts -------
// chunk_hist[c][e] becomes the first sorted position of chunk c's rows of
// expert e; seg_offsets[e] the first position of expert e.  One warp per expert:
// lanes take 32 chunks at a time and scan them with shuffles.
constexpr int kScanThreads = 1024;
__global__ void __launch_bounds__(kScanThreads)
plan_scan_kernel(int* __restrict__ chunk_hist, int n_chunks, int n_experts, int* __restrict__ seg_offsets) {
  __shared__ int s_total[kMaxExperts];
  __shared__ int s_base[kMaxExperts + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_trigger();
  pdl_wait();
  for (int e = warp; e < n_experts; e += kScanThreads / 32) {
    int sum = 0;
    for (int c = lane; c < n_chunks; c += 32) sum += chunk_hist[static_cast<int64_t>(c) * n_experts + e];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if (lane == 0) s_total[e] = sum;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int i = 0; i < n_experts; ++i) { s_base[i] = run; run += s_total[i]; }
    s_base[n_experts] = run;
  }
  __syncthreads();
  if (threadIdx.x <= n_experts) seg_offsets[threadIdx.x] = s_base[threadIdx.x];
  for (int e = warp; e < n_experts; e += kScanThreads / 32) {
    int carry = s_base[e];
    for (int c0 = 0; c0 < n_chunks; c0 += 32) {
      const int c = c0 + lane;
      const int v = c < n_chunks ? chunk_hist[static_cast<int64_t>(c) * n_experts + e] : 0;
      int incl = v;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += up;
      }
      if (c < n_chunks) chunk_hist[static_cast<int64_t>(c) * n_experts + e] = carry + incl - v;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
}

// ---- plan, pass 3: stable rank of every row inside its chunk -----------------
__global__ void __launch_bounds__(kChunkRows)
plan_rank_kernel(const int64_t* __restrict__ flat_idx, int64_t n_rows, int n_experts,
                 const int* __restrict__ chunk_base, int* __restrict__ pos, int* __restrict__ order) {
  constexpr int kWarps = kChunkRows / 32;
  __shared__ int s_warp_count[kWarps][kMaxExperts];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_trigger();
  for (int i = threadIdx.x; i < kWarps * kMaxExperts; i += kChunkRows) (&s_warp_count[0][0])[i] = 0;
  __syncthreads();
  pdl_wait();
  const int64_t r = static_cast<int64_t>(blockIdx.x) * kChunkRows + threadIdx.x;
  int e = -1;
  if (r < n_rows) {
    const int64_t v = flat_idx[r];
    if (v >= 0 && v < n_experts) e = static_cast<int>(v);
  }
  // lanes of this warp holding the same expert (rows are in lane order)
  const unsigned peers = __match_any_sync(0xffffffffu, e);
  const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (e >= 0 && rank_in_warp == 0) s_warp_count[warp][e] = __popc(peers);
  __syncthreads();
  if (e >= 0) {
    int before = 0;
    for (int w = 0; w < warp; ++w) before += s_warp_count[w][e];
    const int p = chunk_base[static_cast<int64_t>(blockIdx.x) * n_experts + e] + before + rank_in_warp;
    pos[r] = p;
    if (order != nullptr) order[p] = static_cast<int>(r);
  } else if (r < n_rows) {
    pos[r] = -1;
  }
}

// ---- plan in one launch, from the router's per-chunk histograms -------------------
// The bf16 router files one histogram per 128 tokens (= one chunk of 256 rows), so passes 1 and 2 are not
// needed: every CTA adds up the (small) table itself.  Keys may be a permutation of the expert ids: with
// `world` > 1 rows are ordered by (owner rank, local slot) of a round-robin expert placement, key(e) =
// (e mod world) * (E / world) + e / world, which is the order the expert-parallel exchange sends them in.
// With K > 0 the row gather is part of the same kernel: `split` CTAs share a chunk, each ranks the whole
// chunk and moves its share of the chunk's tokens.
constexpr int kMaxChunkTable = 16384;  // ints of the per-chunk table one CTA is willing to add up

template <int K>
__global__ void __launch_bounds__(kChunkRows)
plan_chunked_kernel(const int64_t* __restrict__ flat_idx, const int* __restrict__ chunk_hist, int64_t n_rows,
                    int n_experts, int world, int n_chunks, int split, int* __restrict__ pos, int* __restrict__ order,
                    int* __restrict__ seg_offsets, const uint4* __restrict__ x, int row_vec, uint4* __restrict__ out_rows) {
  constexpr int kWarps = kChunkRows / 32;
  constexpr int KK = K > 0 ? K : 1;  // rows per token where the gather is compiled in
  __shared__ int s_total[kMaxExperts];
  __shared__ int s_before[kMaxExperts];
  __shared__ int s_cbase[kMaxExperts];
  __shared__ int s_warp_count[kWarps][kMaxExperts];
  __shared__ int s_pos[kChunkRows];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = blockIdx.x / split, part = blockIdx.x - chunk * split;
  pdl_trigger();
  if (threadIdx.x < kMaxExperts) { s_total[threadIdx.x] = 0; s_before[threadIdx.x] = 0; }
  for (int i = threadIdx.x; i < kWarps * kMaxExperts; i += kChunkRows) (&s_warp_count[0][0])[i] = 0;
  __syncthreads();
  pdl_wait();
  // The first token row of this warp is requested before the plan's loads and barriers, which then run under
  // the row's memory latency (up to kPrefetch 16-byte chunks per lane; longer rows fetch the rest later).
  constexpr int kPrefetch = 5;
  uint4 pre[kPrefetch];
  if (K > 0) {
    const int tokens_per_part = kChunkRows / KK / split;
    const int64_t t = static_cast<int64_t>(chunk) * (kChunkRows / KK) + part * tokens_per_part + warp;
    if (warp < tokens_per_part && t < n_rows / KK) {
      const uint4* src = x + t * row_vec;
#pragma unroll
      for (int j = 0; j < kPrefetch; ++j)
        if (lane + 32 * j < row_vec) pre[j] = ldg_stream16(src + lane + 32 * j);
    }
  }
  // one warp per expert adds up that expert's column of the table: the total and the part in front of this chunk
  for (int ex = warp; ex < n_experts; ex += kWarps) {
    int tot = 0, bef = 0;
    for (int c = lane; c < n_chunks; c += 32) {
      const int v = chunk_hist[c * n_experts + ex];
      tot += v;
      if (c < chunk) bef += v;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      tot += __shfl_xor_sync(0xffffffffu, tot, off);
      bef += __shfl_xor_sync(0xffffffffu, bef, off);
    }
    if (lane == 0) { s_total[ex] = tot; s_before[ex] = bef; }
  }
  const int64_t r = static_cast<int64_t>(chunk) * kChunkRows + threadIdx.x;
  int e = -1;
  if (r < n_rows) {
    const int64_t v = flat_idx[r];
    if (v >= 0 && v < n_experts) e = static_cast<int>(v);
  }
  const unsigned peers = __match_any_sync(0xffffffffu, e);
  const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (e >= 0 && rank_in_warp == 0) s_warp_count[warp][e] = __popc(peers);
  __syncthreads();
  if (threadIdx.x == 0) {
    const int el = n_experts / world;
    int run = 0;
    for (int k = 0; k < n_experts; ++k) {
      const int ek = (k % el) * world + k / el;  // the expert whose key is k
      s_cbase[ek] = run + s_before[ek];
      if (blockIdx.x == 0) seg_offsets[k] = run;
      run += s_total[ek];
    }
    if (blockIdx.x == 0) seg_offsets[n_experts] = run;
  }
  __syncthreads();
  int p = -1;
  if (e >= 0) {
    int before = 0;
    for (int w = 0; w < warp; ++w) before += s_warp_count[w][e];
    p = s_cbase[e] + before + rank_in_warp;
  }
  if (part == 0 && r < n_rows) {
    pos[r] = p;
    if (order != nullptr && p >= 0) order[p] = static_cast<int>(r);
  }
  if (K > 0) {
    s_pos[threadIdx.x] = p;
    __syncthreads();
    const int tokens_per_part = kChunkRows / KK / split;
    const int64_t n_tokens = n_rows / KK;
    for (int i = warp; i < tokens_per_part; i += kWarps) {
      const int tl = part * tokens_per_part + i;  // token inside the chunk
      const int64_t t = static_cast<int64_t>(chunk) * (kChunkRows / KK) + tl;
      if (t >= n_tokens) break;
      int64_t dst[KK];
#pragma unroll
      for (int s = 0; s < K; ++s) dst[s] = static_cast<int64_t>(s_pos[tl * K + s]) * row_vec;
      const uint4* src = x + t * row_vec;
      int c0 = lane;
      if (i == warp) {  // this warp's first token: its head is already in registers
#pragma unroll
        for (int j = 0; j < kPrefetch; ++j) {
          const int c = lane + 32 * j;
          if (c < row_vec) {
#pragma unroll
            for (int s = 0; s < K; ++s)
              if (dst[s] >= 0) stg_stream16(out_rows + dst[s] + c, pre[j]);
          }
        }
        c0 = lane + 32 * kPrefetch;
      }
#pragma unroll 4
      for (int c = c0; c < row_vec; c += 32) {
        const uint4 v = ldg_stream16(src + c);
#pragma unroll
        for (int s = 0; s < K; ++s)
          if (dst[s] >= 0) stg_stream16(out_rows + dst[s] + c, v);
      }
    }
  }
}

// ---- row gather: out_rows[pos[t*k+s]] = x[t] ---------------------------------
template <int K>
__global__ void __launch_bounds__(256)
permute_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ pos, int64_t n_tokens, int row_vec,
                    uint4* __restrict__ out) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * 8 + warp;
  pdl_trigger();
  pdl_wait();
  if (t >= n_tokens) return;
  int64_t dst[K];
#pragma unroll
  for (int s = 0; s < K; ++s) dst[s] = static_cast<int64_t>(pos[t * K + s]) * row_vec;
  const uint4* src = x + t * row_vec;
#pragma unroll 4
  for (int c = lane; c < row_vec; c += 32) {
    const uint4 v = ldg_stream16(src + c);
#pragma unroll
    for (int s = 0; s < K; ++s)
      if (dst[s] >= 0) stg_stream16(out + dst[s] + c, v);
  }
}

// ---- inverse gather + weighted pair sum ---------------------------------------
template <typename T>
struct Vec16;
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int kElems = 8;
  __device__ static void to_float(const uint4& v, float* f) {
    f[0] = bf16lo_to_f32(v.x); f[1] = bf16hi_to_f32(v.x); f[2] = bf16lo_to_f32(v.y); f[3] = bf16hi_to_f32(v.y);
    f[4] = bf16lo_to_f32(v.z); f[5] = bf16hi_to_f32(v.z); f[6] = bf16lo_to_f32(v.w); f[7] = bf16hi_to_f32(v.w);
  }
  __device__ static uint4 from_float(const float* f) {
    return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
  }
};
template <>
struct Vec16<float> {
  static constexpr int kElems = 4;
  __device__ static void to_float(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
  __device__ static uint4 from_float(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
};

template <typename T, bool kGlue>
__global__ void __launch_bounds__(256, kGlue ? 4 : 6)
unpermute_combine_kernel(const uint4* __restrict__ src0, const int* __restrict__ idx0, int idx0_stride,
                         const uint4* __restrict__ src1, const int* __restrict__ idx1, int idx1_stride,
                         const float* __restrict__ w0, const float* __restrict__ w1, int w_stride,
                         const uint4* __restrict__ addend, const uint4* __restrict__ resid, const uint4* __restrict__ gate,
                         int tokens_per_sample, int64_t n_tokens, int row_vec, uint4* __restrict__ out) {
  constexpr int EL = Vec16<T>::kElems;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * 8 + warp;
  pdl_trigger();
  pdl_wait();
  if (t >= n_tokens) return;
  const int64_t i0 = idx0 ? static_cast<int64_t>(idx0[t * idx0_stride]) : t;
  const int64_t i1 = src1 ? (idx1 ? static_cast<int64_t>(idx1[t * idx1_stride]) : t) : -1;
  const float a0 = w0 ? w0[t * w_stride] : 1.f;
  const float a1 = w1 ? w1[t * w_stride] : 1.f;
  const uint4* p0 = (i0 >= 0) ? src0 + i0 * row_vec : nullptr;
  const uint4* p1 = (i1 >= 0) ? src1 + i1 * row_vec : nullptr;
  const uint4* pa = addend ? addend + t * row_vec : nullptr;
  // the gated residual of the DiT block: out = resid + gate[sample of t] * (the sum above)
  const uint4* pr = (kGlue && resid) ? resid + t * row_vec : nullptr;
  const uint4* pg = (kGlue && gate) ? gate + (t / tokens_per_sample) * row_vec : nullptr;
  uint4* po = out + t * row_vec;
#pragma unroll 2
  for (int c = lane; c < row_vec; c += 32) {
    float acc[EL];
#pragma unroll
    for (int j = 0; j < EL; ++j) acc[j] = 0.f;
    if (p0) {
      float f[EL];
      Vec16<T>::to_float(ldg_stream16(p0 + c), f);
#pragma unroll
      for (int j = 0; j < EL; ++j) acc[j] = a0 * f[j];
    }
    if (p1) {
      float f[EL];
      Vec16<T>::to_float(ldg_stream16(p1 + c), f);
#pragma unroll
      for (int j = 0; j < EL; ++j) acc[j] = fmaf(a1, f[j], acc[j]);
    }
    if (pa) {
      float f[EL];
      Vec16<T>::to_float(ldg_stream16(pa + c), f);
#pragma unroll
      for (int j = 0; j < EL; ++j) acc[j] += f[j];
    }
    if (kGlue && pg) {
      float f[EL];
      Vec16<T>::to_float(__ldg(pg + c), f);
#pragma unroll
      for (int j = 0; j < EL; ++j) acc[j] *= f[j];
    }
    if (kGlue && pr) {
      float f[EL];
      Vec16<T>::to_float(ldg_stream16(pr + c), f);
#pragma unroll
      for (int j = 0; j < EL; ++j) acc[j] += f[j];
    }
    stg_stream16(po + c, Vec16<T>::from_float(acc));
  }
}

// ---- SwiGLU weight packing ------------------------------------------------------
__global__ void pack_w13_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up, int row_vec, int ffn,
                                int64_t out_rows, uint4* __restrict__ out) {
  const int64_t total = out_rows * row_vec;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / row_vec;
    const int c = static_cast<int>(i - row * row_vec);
    const int64_t blk = row / 256;
    const int within = static_cast<int>(row - blk * 256);
    const int64_t src_row = blk * 128 + (within & 127);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (src_row < ffn) v = (within < 128 ? gate : up)[src_row * row_vec + c];
    out[i] = v;
  }
}

}  // namespace

extern "C" size_t dice_permute_scratch_bytes(int64_t n_rows, int n_experts) {
  if (n_rows < 0 || n_experts <= 0) return 0;
  const int64_t chunks = (n_rows + kChunkRows - 1) / kChunkRows;
  return static_cast<size_t>((chunks > 0 ? chunks : 1) * n_experts) * sizeof(int);
}

extern "C" int dice_permute_plan(const int64_t* flat_idx, int64_t n_rows, int n_experts, void* scratch,
                                 size_t scratch_bytes, int32_t* out_pos, int32_t* out_order,
                                 int32_t* out_seg_offsets, void* stream) {
  DICE_CHECK_ARG(n_rows >= 0 && out_seg_offsets != nullptr, DICE_ERR_ARG);
  DICE_CHECK_ARG(n_experts >= 1 && n_experts <= kMaxExperts, DICE_ERR_SHAPE);
  DICE_CHECK_ARG(n_rows <= 0x7fffffffLL - kChunkRows, DICE_ERR_LIMIT);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n_rows == 0) {
    DICE_CUDA_OK(cudaMemsetAsync(out_seg_offsets, 0, sizeof(int32_t) * (n_experts + 1), s));
    return DICE_OK;
  }
  DICE_CHECK_ARG(flat_idx && scratch && out_pos, DICE_ERR_ARG);
  DICE_CHECK_ARG(scratch_bytes >= dice_permute_scratch_bytes(n_rows, n_experts), DICE_ERR_SCRATCH);
  const int chunks = static_cast<int>((n_rows + kChunkRows - 1) / kChunkRows);
  int* chunk_hist = static_cast<int*>(scratch);
  DICE_CUDA_OK(dice_launch(plan_count_kernel, dim3(chunks), dim3(kChunkRows), 0, s, flat_idx, n_rows, n_experts, chunk_hist));
  DICE_CUDA_OK(dice_launch(plan_scan_kernel, dim3(1), dim3(kScanThreads), 0, s, chunk_hist, chunks, n_experts,
                           out_seg_offsets));
  DICE_CUDA_OK(dice_launch(plan_rank_kernel, dim3(chunks), dim3(kChunkRows), 0, s, flat_idx, n_rows, n_experts,
                           chunk_hist, out_pos, out_order));
  return DICE_OK;
}

// Device address of g_plan_static_scratch on the current device, looked up once per device.
static int static_plan_scratch(int** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static int* addr[kMaxDevices] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return DICE_ERR_CUDA;
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_plan_static_scratch) != cudaSuccess || p == nullptr) return DICE_ERR_CUDA;
    addr[dev] = static_cast<int*>(p);
  }
  *out = addr[dev];
  return DICE_OK;
}

extern "C" int dice_permute_plan_static(const int64_t* flat_idx, int64_t n_rows, int n_experts, int32_t* out_pos,
                                        int32_t* out_order, int32_t* out_seg_offsets, void* stream) {
  DICE_CHECK_ARG(n_rows >= 0 && out_seg_offsets != nullptr, DICE_ERR_ARG);
  DICE_CHECK_ARG(n_experts >= 1 && n_experts <= kMaxExperts, DICE_ERR_SHAPE);
  const int64_t chunks = (n_rows + kChunkRows - 1) / kChunkRows;
  DICE_CHECK_ARG(chunks * n_experts <= DICE_PLAN_STATIC_MAX_INTS, DICE_ERR_LIMIT);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n_rows == 0) {
    DICE_CUDA_OK(cudaMemsetAsync(out_seg_offsets, 0, sizeof(int32_t) * (n_experts + 1), s));
    return DICE_OK;
  }
  DICE_CHECK_ARG(flat_idx && out_pos, DICE_ERR_ARG);
  int* chunk_hist = nullptr;
  const int rc = static_plan_scratch(&chunk_hist);
  if (rc != DICE_OK) return rc;
  // pass 1 overwrites every cell the later passes read, so nothing has to be cleared between calls
  const int n_chunks = static_cast<int>(chunks);
  DICE_CUDA_OK(dice_launch(plan_count_kernel, dim3(n_chunks), dim3(kChunkRows), 0, s, flat_idx, n_rows, n_experts,
                           chunk_hist));
  DICE_CUDA_OK(dice_launch(plan_scan_kernel, dim3(1), dim3(kScanThreads), 0, s, chunk_hist, n_chunks, n_experts,
                           out_seg_offsets));
  DICE_CUDA_OK(dice_launch(plan_rank_kernel, dim3(n_chunks), dim3(kChunkRows), 0, s, flat_idx, n_rows, n_experts,
                           chunk_hist, out_pos, out_order));
  return DICE_OK;
}

extern "C" int dice_permute_plan_chunked(const int64_t* flat_idx, const int32_t* chunk_hist, int64_t n_rows,
                                         int n_experts, int world, int32_t* out_pos, int32_t* out_order,
                                         int32_t* out_seg_offsets, const void* x, int k, int hidden, int dtype,
                                         void* out_rows, void* stream) {
  DICE_CHECK_ARG(n_rows >= 0 && out_seg_offsets != nullptr, DICE_ERR_ARG);
  DICE_CHECK_ARG(n_experts >= 1 && n_experts <= kMaxExperts && world >= 1 && n_experts % world == 0, DICE_ERR_SHAPE);
  const int64_t chunks = (n_rows + kChunkRows - 1) / kChunkRows;
  DICE_CHECK_ARG(chunks * n_experts <= kMaxChunkTable, DICE_ERR_LIMIT);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n_rows == 0) {
    DICE_CUDA_OK(cudaMemsetAsync(out_seg_offsets, 0, sizeof(int32_t) * (n_experts + 1), s));
    return DICE_OK;
  }
  DICE_CHECK_ARG(flat_idx && chunk_hist && out_pos, DICE_ERR_ARG);
  const int n_chunks = static_cast<int>(chunks);
  if (x == nullptr) {
    DICE_CUDA_OK(dice_launch(plan_chunked_kernel<0>, dim3(n_chunks), dim3(kChunkRows), 0, s, flat_idx, chunk_hist, n_rows,
                             n_experts, world, n_chunks, 1, out_pos, out_order, out_seg_offsets,
                             static_cast<const uint4*>(nullptr), 0, static_cast<uint4*>(nullptr)));
    return DICE_OK;
  }
  DICE_CHECK_ARG(k == 1 || k == 2, DICE_ERR_SHAPE);
  DICE_CHECK_ARG(n_rows % k == 0 && hidden > 0 && out_rows != nullptr, DICE_ERR_ARG);
  const size_t es = dice_dtype_size(dtype);
  DICE_CHECK_ARG(es != 0, DICE_ERR_DTYPE);
  DICE_CHECK_ARG((hidden * es) % 16 == 0, DICE_ERR_SHAPE);
  DICE_CHECK_ARG(dice_aligned16(x) && dice_aligned16(out_rows), DICE_ERR_ALIGN);
  const int row_vec = static_cast<int>(hidden * es / 16);
  const int split = 16;  // CTAs per chunk: 8 (k = 2) or 16 (k = 1) tokens each, one or two per warp
  if (k == 2)
    DICE_CUDA_OK(dice_launch(plan_chunked_kernel<2>, dim3(n_chunks * split), dim3(kChunkRows), 0, s, flat_idx, chunk_hist,
                             n_rows, n_experts, world, n_chunks, split, out_pos, out_order, out_seg_offsets,
                             static_cast<const uint4*>(x), row_vec, static_cast<uint4*>(out_rows)));
  else
    DICE_CUDA_OK(dice_launch(plan_chunked_kernel<1>, dim3(n_chunks * split), dim3(kChunkRows), 0, s, flat_idx, chunk_hist,
                             n_rows, n_experts, world, n_chunks, split, out_pos, out_order, out_seg_offsets,
                             static_cast<const uint4*>(x), row_vec, static_cast<uint4*>(out_rows)));
  return DICE_OK;
}

extern "C" int dice_permute_rows(const void* x, const int32_t* pos, int64_t n_tokens, int k, int hidden, int dtype,
                                 void* out_rows, void* stream) {
  DICE_CHECK_ARG(n_tokens >= 0 && hidden > 0, DICE_ERR_ARG);
  DICE_CHECK_ARG(k == 1 || k == 2, DICE_ERR_SHAPE);
  const size_t es = dice_dtype_size(dtype);
  DICE_CHECK_ARG(es != 0, DICE_ERR_DTYPE);
  DICE_CHECK_ARG((hidden * es) % 16 == 0, DICE_ERR_SHAPE);
  if (n_tokens == 0) return DICE_OK;
  DICE_CHECK_ARG(x && pos && out_rows, DICE_ERR_ARG);
  DICE_CHECK_ARG(dice_aligned16(x) && dice_aligned16(out_rows), DICE_ERR_ALIGN);
  const int row_vec = static_cast<int>(hidden * es / 16);
  const int64_t blocks = (n_tokens + 7) / 8;
  DICE_CHECK_ARG(blocks <= 0x7fffffffLL, DICE_ERR_LIMIT);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(static_cast<unsigned>(blocks));
  if (k == 2)
    DICE_CUDA_OK(dice_launch(permute_rows_kernel<2>, grid, dim3(256), 0, s, static_cast<const uint4*>(x), pos, n_tokens,
                             row_vec, static_cast<uint4*>(out_rows)));
  else
    DICE_CUDA_OK(dice_launch(permute_rows_kernel<1>, grid, dim3(256), 0, s, static_cast<const uint4*>(x), pos, n_tokens,
                             row_vec, static_cast<uint4*>(out_rows)));
  return DICE_OK;
}

extern "C" int dice_unpermute_combine(const void* src0, const int32_t* idx0, int idx0_stride, const void* src1,
                                      const int32_t* idx1, int idx1_stride, const float* w0, const float* w1,
                                      int w_stride, const void* addend, const void* resid, const void* gate,
                                      int tokens_per_sample, int64_t n_tokens, int hidden, int dtype, void* out,
                                      void* stream) {
  DICE_CHECK_ARG(n_tokens >= 0 && hidden > 0, DICE_ERR_ARG);
  DICE_CHECK_ARG(gate == nullptr || tokens_per_sample > 0, DICE_ERR_ARG);
  const size_t es = dice_dtype_size(dtype);
  DICE_CHECK_ARG(es != 0, DICE_ERR_DTYPE);
  DICE_CHECK_ARG((hidden * es) % 16 == 0, DICE_ERR_SHAPE);
  if (n_tokens == 0) return DICE_OK;
  DICE_CHECK_ARG(src0 && out, DICE_ERR_ARG);
  DICE_CHECK_ARG(dice_aligned16(src0) && dice_aligned16(out) && dice_aligned16(src1) && dice_aligned16(addend) &&
                     dice_aligned16(resid) && dice_aligned16(gate),
                 DICE_ERR_ALIGN);
  if (tokens_per_sample <= 0) tokens_per_sample = 1;
  const int row_vec = static_cast<int>(hidden * es / 16);
  const int64_t blocks = (n_tokens + 7) / 8;
  DICE_CHECK_ARG(blocks <= 0x7fffffffLL, DICE_ERR_LIMIT);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(static_cast<unsigned>(blocks));
  const bool glue = resid != nullptr || gate != nullptr;
#define DICE_LAUNCH_COMBINE(T, G)                                                                                        \
  DICE_CUDA_OK(dice_launch(unpermute_combine_kernel<T, G>, grid, dim3(256), 0, s, static_cast<const uint4*>(src0), idx0,  \
                           idx0_stride, static_cast<const uint4*>(src1), idx1, idx1_stride, w0, w1, w_stride,            \
                           static_cast<const uint4*>(addend), static_cast<const uint4*>(resid),                          \
                           static_cast<const uint4*>(gate), tokens_per_sample, n_tokens, row_vec, static_cast<uint4*>(out)))
  if (dtype == DICE_BF16) {
    if (glue) DICE_LAUNCH_COMBINE(__nv_bfloat16, true);
    else DICE_LAUNCH_COMBINE(__nv_bfloat16, false);
  } else {
    if (glue) DICE_LAUNCH_COMBINE(float, true);
    else DICE_LAUNCH_COMBINE(float, false);
  }
#undef DICE_LAUNCH_COMBINE
  return DICE_OK;
}

extern "C" int64_t dice_w13_rows(int ffn) { return ffn <= 0 ? 0 : (static_cast<int64_t>(ffn) + 127) / 128 * 256; }

extern "C" int dice_pack_w13(const void* gate_proj, const void* up_proj, int hidden, int ffn, int dtype,
                             void* out_w13, void* stream) {
  DICE_CHECK_ARG(gate_proj && up_proj && out_w13 && hidden > 0 && ffn > 0, DICE_ERR_ARG);
  const size_t es = dice_dtype_size(dtype);
  DICE_CHECK_ARG(es != 0, DICE_ERR_DTYPE);
  DICE_CHECK_ARG((hidden * es) % 16 == 0, DICE_ERR_SHAPE);
  DICE_CHECK_ARG(dice_aligned16(gate_proj) && dice_aligned16(up_proj) && dice_aligned16(out_w13), DICE_ERR_ALIGN);
  const int row_vec = static_cast<int>(hidden * es / 16);
  const int64_t out_rows = dice_w13_rows(ffn);
  const int64_t total = out_rows * row_vec;
  const int blocks = static_cast<int>(total / 256 + 1 < 4096 ? total / 256 + 1 : 4096);
  dice_count_launch();
  pack_w13_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(gate_proj), static_cast<const uint4*>(up_proj), row_vec, ffn, out_rows,
      static_cast<uint4*>(out_w13));
  return cudaGetLastError() == cudaSuccess ? DICE_OK : DICE_ERR_CUDA;
}
