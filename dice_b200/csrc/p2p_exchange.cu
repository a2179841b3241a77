// Expert-parallel exchange over NVLink peer memory, without NCCL and without a
// host round trip.
//
// Every rank owns, per exchange slot, a few buffers that its peers map through
// CUDA IPC: a count matrix [W][E], three flag arrays [W] and two row buffers
// (dispatch receive, combine receive).  A rank never reads peer memory; it only
// WRITES into it (coalesced 16-byte stores over NVLink) and then raises a flag
// there.  Four kernels, all launched on the caller's stream:
//
//   1. ep_counts_kernel    publish this rank's per-(owner, slot) row counts in
//                          every peer's matrix, wait for all rows, derive where
//                          this rank's rows land in each peer's buffers and how
//                          the rows it will receive are segmented;
//   2. ep_dispatch_kernel  the row gather of the permutation fused with the
//                          dispatch: each (token, slot) row is written straight
//                          into its expert owner's receive buffer;
//   3. ep_wait_kernel      wait until every source has raised its "rows written"
//                          flag (before the expert FFN / before the combine);
//   4. ep_return_kernel    write the expert outputs back into the token owners'
//                          combine buffers, in the order they were sent.
//
// Ordering: writers fence at system scope, the last CTA of a grid raises the
// flags with release stores; waiters poll with acquire loads.  Every wait is
// bounded by wall time; on expiry a status code is recorded and the kernel
// returns (results of that call are then undefined, the context stays usable).
#include <cuda.h>
#include <string.h>

#include "common.cuh"

namespace {

constexpr int kMaxRanks = 16;
constexpr int kMaxKeys = 64;  // experts
constexpr uint64_t kPeerWaitLimitNs = 2000ull * 1000ull * 1000ull;

struct PeerTable {
  void* ptr[kMaxRanks];
};

__device__ __forceinline__ uint64_t timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// true when *flag reached `seq` within the time limit
__device__ bool wait_flag(const uint32_t* flag, uint32_t seq, uint32_t* status, uint32_t code) {
  const uint64_t t0 = timer_ns();
  uint32_t spins = 0;
  for (;;) {
    if (static_cast<int32_t>(ld_acquire_sys(flag) - seq) >= 0) return true;
    if ((++spins & 63u) == 0) {
      if (timer_ns() - t0 > kPeerWaitLimitNs) {
        if (status != nullptr) atomicCAS(status, 0u, code);
        return false;
      }
      __nanosleep(200);
    }
  }
}

// Layout of the per-slot meta block this rank derives in ep_counts_kernel (int32):
//   [0, W)            send_base[d]   first row of this rank's block in peer d's dispatch buffer
//   [W, 2W)           back_base[s]   first row of this rank's block in peer s's combine buffer
//   [2W, 3W+1)        src_off[s]     first row received from source s (W+1 entries)
//   [3W+1, 3W+2+W*El) seg_off[...]   offsets of the (source, slot) segments of the receive buffer
//   then              total_recv, overflow
__host__ __device__ inline int meta_ints(int w, int el) { return 3 * w + 1 + w * el + 1 + 2; }

// ---- 1. counts ---------------------------------------------------------------------
__global__ void __launch_bounds__(256)
ep_counts_kernel(const int* __restrict__ seg_offsets,  // [E+1] this rank's key-sorted segments (key = owner*El + slot)
                 PeerTable matrices,                    // peer d: int32 [W][E]
                 PeerTable flags,                       // peer d: uint32 [W]
                 int* __restrict__ my_matrix, const uint32_t* __restrict__ my_flags, int* __restrict__ meta,
                 int rank, int world, int n_keys, int capacity_rows, uint32_t seq, uint32_t* status) {
  __shared__ int s_cnt[kMaxRanks][kMaxKeys];
  __shared__ int s_ok;
  const int el = n_keys / world;
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x == 0) s_ok = 1;
  // publish my row everywhere (my own matrix included)
  for (int i = threadIdx.x; i < world * n_keys; i += blockDim.x) {
    const int d = i / n_keys, e = i - d * n_keys;
    static_cast<int*>(matrices.ptr[d])[rank * n_keys + e] = seg_offsets[e + 1] - seg_offsets[e];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world) st_release_sys(static_cast<uint32_t*>(flags.ptr[threadIdx.x]) + rank, seq);
  // wait for every source's row
  if (threadIdx.x < world) {
    if (!wait_flag(my_flags + threadIdx.x, seq, status, DICE_STATUS_WAIT_PEER_COUNTS)) s_ok = 0;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < world * n_keys; i += blockDim.x)
    s_cnt[i / n_keys][i % n_keys] = s_ok ? my_matrix[i] : 0;
  __syncthreads();
  if (threadIdx.x == 0) {
    int* send_base = meta;
    int* back_base = meta + world;
    int* src_off = meta + 2 * world;
    int* seg_off = meta + 3 * world + 1;
    // rows source s sends to owner d
    auto block_rows = [&](int s, int d) {
      int n = 0;
      for (int i = 0; i < el; ++i) n += s_cnt[s][d * el + i];
      return n;
    };
    for (int d = 0; d < world; ++d) {
      int base = 0;
      for (int s = 0; s < rank; ++s) base += block_rows(s, d);
      send_base[d] = base;
    }
    for (int s = 0; s < world; ++s) {
      int base = 0;
      for (int d = 0; d < rank; ++d) base += block_rows(s, d);
      back_base[s] = base;
    }
    int run = 0, seg = 0;
    for (int s = 0; s < world; ++s) {
      src_off[s] = run;
      for (int i = 0; i < el; ++i) {
        seg_off[seg++] = run;
        run += s_cnt[s][rank * el + i];
      }
    }
    src_off[world] = run;
    seg_off[seg] = run;
    int* tail = seg_off + world * el + 1;
    tail[0] = run;
    tail[1] = run > capacity_rows ? 1 : 0;
    if (run > capacity_rows) {
      if (status != nullptr) atomicCAS(status, 0u, DICE_STATUS_EXCHANGE_OVERFLOW);
      // keep the FFN inside the buffer: drop the segments (the call's result is invalid and flagged)
      for (int i = 0; i <= world * el; ++i) seg_off[i] = 0;
    }
  }
}

// raise `flag[rank] = seq` on every peer once the whole grid has finished writing
__device__ __forceinline__ void signal_when_grid_done(unsigned int* done_counter, PeerTable flags, int rank, int world,
                                                      uint32_t seq) {
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(done_counter, 1u);
    s_last = prev == gridDim.x - 1;
  }
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (threadIdx.x < world) st_release_sys(static_cast<uint32_t*>(flags.ptr[threadIdx.x]) + rank, seq);
    if (threadIdx.x == 0) *done_counter = 0;  // ready for the next launch on this stream
  }
}

// ---- 2. dispatch: permutation gather fused with the push into the owners' buffers --------
template <int K>
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const uint4* __restrict__ x, const int* __restrict__ pos, const int* __restrict__ seg_offsets,
                   const int* __restrict__ meta, PeerTable recv_bufs, PeerTable flags, unsigned int* done_counter,
                   int64_t n_tokens, int row_vec, int rank, int world, int el, int capacity_rows, uint32_t seq,
                   uint32_t* status) {
  __shared__ int s_first[kMaxRanks + 1];  // first sorted position of each owner's block
  __shared__ int s_base[kMaxRanks];
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x <= world) s_first[threadIdx.x] = seg_offsets[threadIdx.x * el];
  if (threadIdx.x < world) s_base[threadIdx.x] = meta[threadIdx.x];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * 8 + warp; t < n_tokens; t += static_cast<int64_t>(gridDim.x) * 8) {
    uint4* dst[K];
#pragma unroll
    for (int s = 0; s < K; ++s) {
      dst[s] = nullptr;
      const int p = pos[t * K + s];
      if (p >= 0) {
        int d = 0;
        while (d + 1 < world && p >= s_first[d + 1]) ++d;
        const int row = s_base[d] + (p - s_first[d]);
        if (row < capacity_rows) dst[s] = static_cast<uint4*>(recv_bufs.ptr[d]) + static_cast<int64_t>(row) * row_vec;
        else if (lane == 0 && status != nullptr) atomicCAS(status, 0u, DICE_STATUS_EXCHANGE_OVERFLOW);
      }
    }
    const uint4* src = x + t * row_vec;
#pragma unroll 4
    for (int c = lane; c < row_vec; c += 32) {
      const uint4 v = ldg_stream16(src + c);
#pragma unroll
      for (int s = 0; s < K; ++s)
        if (dst[s] != nullptr) dst[s][c] = v;
    }
  }
  signal_when_grid_done(done_counter, flags, rank, world, seq);
}

// ---- 3. wait for all sources ------------------------------------------------------------
__global__ void ep_wait_kernel(const uint32_t* __restrict__ my_flags, int world, uint32_t seq, uint32_t* status,
                               uint32_t code) {
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x < world) wait_flag(my_flags + threadIdx.x, seq, status, code);
}

// ---- 4. return: expert outputs go back to the token owners --------------------------------
__global__ void __launch_bounds__(256)
ep_return_kernel(const uint4* __restrict__ rows, const int* __restrict__ meta, PeerTable back_bufs, PeerTable flags,
                 unsigned int* done_counter, int row_vec, int rank, int world, int back_capacity_rows, uint32_t seq,
                 uint32_t* status) {
  __shared__ int s_src_off[kMaxRanks + 1];
  __shared__ int s_back[kMaxRanks];
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x <= world) s_src_off[threadIdx.x] = meta[2 * world + threadIdx.x];
  if (threadIdx.x < world) s_back[threadIdx.x] = meta[world + threadIdx.x];
  __syncthreads();
  const int total = s_src_off[world];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int64_t r = static_cast<int64_t>(blockIdx.x) * 8 + warp; r < total; r += static_cast<int64_t>(gridDim.x) * 8) {
    int s = 0;
    while (s + 1 < world && r >= s_src_off[s + 1]) ++s;
    const int row = s_back[s] + static_cast<int>(r - s_src_off[s]);
    if (row >= back_capacity_rows) {
      if (lane == 0 && status != nullptr) atomicCAS(status, 0u, DICE_STATUS_EXCHANGE_OVERFLOW);
      continue;
    }
    uint4* dst = static_cast<uint4*>(back_bufs.ptr[s]) + static_cast<int64_t>(row) * row_vec;
    const uint4* src = rows + r * row_vec;
#pragma unroll 4
    for (int c = lane; c < row_vec; c += 32) dst[c] = ldg_stream16(src + c);
  }
  signal_when_grid_done(done_counter, flags, rank, world, seq);
}

int fill_table(PeerTable* t, const void* const* ptrs, int world) {
  if (ptrs == nullptr || world < 1 || world > kMaxRanks) return DICE_ERR_ARG;
  for (int i = 0; i < kMaxRanks; ++i) t->ptr[i] = i < world ? const_cast<void*>(ptrs[i]) : nullptr;
  for (int i = 0; i < world; ++i)
    if (t->ptr[i] == nullptr) return DICE_ERR_ARG;
  return DICE_OK;
}

}  // namespace

extern "C" int dice_ep_meta_ints(int world, int n_local_experts) {
  if (world < 1 || world > kMaxRanks || n_local_experts < 1) return 0;
  return meta_ints(world, n_local_experts);
}

extern "C" int dice_ep_exchange_counts(const int32_t* seg_offsets, const void* const* peer_matrices,
                                       const void* const* peer_flags, int32_t* meta, int rank, int world,
                                       int n_experts, int capacity_rows, uint32_t seq, uint32_t* status,
                                       void* stream) {
  DICE_CHECK_ARG(seg_offsets && meta && world >= 1 && rank >= 0 && rank < world, DICE_ERR_ARG);
  DICE_CHECK_ARG(world <= kMaxRanks && n_experts <= kMaxKeys && n_experts % world == 0, DICE_ERR_SHAPE);
  PeerTable m, f;
  int rc = fill_table(&m, peer_matrices, world);
  if (rc != DICE_OK) return rc;
  rc = fill_table(&f, peer_flags, world);
  if (rc != DICE_OK) return rc;
  DICE_CUDA_OK(dice_launch(ep_counts_kernel, dim3(1), dim3(256), 0, static_cast<cudaStream_t>(stream), seg_offsets, m, f,
                           static_cast<int*>(m.ptr[rank]), static_cast<const uint32_t*>(f.ptr[rank]), meta, rank, world,
                           n_experts, capacity_rows, seq, status));
  return DICE_OK;
}

extern "C" int dice_ep_dispatch_rows(const void* x, const int32_t* pos, const int32_t* seg_offsets,
                                     const int32_t* meta, const void* const* peer_recv, const void* const* peer_flags,
                                     uint32_t* done_counter, int64_t n_tokens, int k, int hidden, int dtype, int rank,
                                     int world, int n_experts, int capacity_rows, uint32_t seq, int max_ctas,
                                     uint32_t* status, void* stream) {
  DICE_CHECK_ARG(n_tokens >= 0 && hidden > 0 && done_counter && meta && seg_offsets, DICE_ERR_ARG);
  DICE_CHECK_ARG(k == 1 || k == 2, DICE_ERR_SHAPE);
  DICE_CHECK_ARG(world >= 1 && world <= kMaxRanks && n_experts % world == 0, DICE_ERR_SHAPE);
  const size_t es = dice_dtype_size(dtype);
  DICE_CHECK_ARG(es != 0, DICE_ERR_DTYPE);
  DICE_CHECK_ARG((hidden * es) % 16 == 0, DICE_ERR_SHAPE);
  DICE_CHECK_ARG(n_tokens == 0 || (x && pos && dice_aligned16(x)), DICE_ERR_ARG);
  PeerTable r, f;
  int rc = fill_table(&r, peer_recv, world);
  if (rc != DICE_OK) return rc;
  rc = fill_table(&f, peer_flags, world);
  if (rc != DICE_OK) return rc;
  const int row_vec = static_cast<int>(hidden * es / 16);
  int64_t blocks = (n_tokens + 7) / 8;
  if (blocks < 1) blocks = 1;  // the flags are raised even when this rank has nothing to send
  if (max_ctas > 0 && blocks > max_ctas) blocks = max_ctas;  // a small grid leaves the SMs to a concurrent GEMM
  DICE_CHECK_ARG(blocks <= 0x7fffffffLL, DICE_ERR_LIMIT);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int el = n_experts / world;
  const dim3 grid(static_cast<unsigned>(blocks));
  if (k == 2)
    DICE_CUDA_OK(dice_launch(ep_dispatch_kernel<2>, grid, dim3(256), 0, s, static_cast<const uint4*>(x), pos, seg_offsets,
                             meta, r, f, done_counter, n_tokens, row_vec, rank, world, el, capacity_rows, seq, status));
  else
    DICE_CUDA_OK(dice_launch(ep_dispatch_kernel<1>, grid, dim3(256), 0, s, static_cast<const uint4*>(x), pos, seg_offsets,
                             meta, r, f, done_counter, n_tokens, row_vec, rank, world, el, capacity_rows, seq, status));
  return DICE_OK;
}

extern "C" int dice_ep_wait_flags(const uint32_t* my_flags, int world, uint32_t seq, int what, uint32_t* status,
                                  void* stream) {
  DICE_CHECK_ARG(my_flags && world >= 1 && world <= kMaxRanks, DICE_ERR_ARG);
  const uint32_t code = what == 0 ? DICE_STATUS_WAIT_PEER_DISPATCH : DICE_STATUS_WAIT_PEER_COMBINE;
  DICE_CUDA_OK(dice_launch(ep_wait_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), my_flags, world, seq,
                           status, code));
  return DICE_OK;
}

extern "C" int dice_ep_return_rows(const void* rows, const int32_t* meta, const void* const* peer_back,
                                   const void* const* peer_flags, uint32_t* done_counter, int hidden, int dtype,
                                   int rank, int world, int back_capacity_rows, int max_rows, uint32_t seq,
                                   int max_ctas, uint32_t* status, void* stream) {
  DICE_CHECK_ARG(rows && meta && done_counter && hidden > 0 && max_rows >= 0, DICE_ERR_ARG);
  DICE_CHECK_ARG(world >= 1 && world <= kMaxRanks, DICE_ERR_SHAPE);
  const size_t es = dice_dtype_size(dtype);
  DICE_CHECK_ARG(es != 0, DICE_ERR_DTYPE);
  DICE_CHECK_ARG((hidden * es) % 16 == 0 && dice_aligned16(rows), DICE_ERR_SHAPE);
  PeerTable b, f;
  int rc = fill_table(&b, peer_back, world);
  if (rc != DICE_OK) return rc;
  rc = fill_table(&f, peer_flags, world);
  if (rc != DICE_OK) return rc;
  const int row_vec = static_cast<int>(hidden * es / 16);
  int64_t blocks = (static_cast<int64_t>(max_rows) + 7) / 8;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 16) blocks = 148 * 16;  // grid-stride over the rows actually received
  if (max_ctas > 0 && blocks > max_ctas) blocks = max_ctas;
  DICE_CUDA_OK(dice_launch(ep_return_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0,
                           static_cast<cudaStream_t>(stream), static_cast<const uint4*>(rows), meta, b, f, done_counter,
                           row_vec, rank, world, back_capacity_rows, seq, status));
  return DICE_OK;
}

// ---- CUDA IPC plumbing (set-up time only) ---------------------------------------------------
extern "C" int dice_ipc_export(const void* ptr, uint8_t* out_handle64, uint64_t* out_offset) {
  DICE_CHECK_ARG(ptr && out_handle64 && out_offset, DICE_ERR_ARG);
  typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q) != cudaSuccess || fn == nullptr)
    return DICE_ERR_CUDA;
  CUdeviceptr base = 0;
  size_t size = 0;
  if (reinterpret_cast<RangeFn>(fn)(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS) return DICE_ERR_CUDA;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)) != cudaSuccess) return DICE_ERR_CUDA;
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(out_handle64, &h, 64);
  *out_offset = reinterpret_cast<CUdeviceptr>(ptr) - base;
  return DICE_OK;
}

extern "C" int dice_ipc_import(const uint8_t* handle64, uint64_t offset, void** out_ptr) {
  DICE_CHECK_ARG(handle64 && out_ptr, DICE_ERR_ARG);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* base = nullptr;
  if (cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return DICE_ERR_CUDA;
  }
  *out_ptr = static_cast<uint8_t*>(base) + offset;
  return DICE_OK;
}

extern "C" int dice_ipc_close(void* imported_ptr, uint64_t offset) {
  DICE_CHECK_ARG(imported_ptr, DICE_ERR_ARG);
  return cudaIpcCloseMemHandle(static_cast<uint8_t*>(imported_ptr) - offset) == cudaSuccess ? DICE_OK : DICE_ERR_CUDA;
}
