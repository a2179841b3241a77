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
#include <stdlib.h>
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


// ---- bulk-copy variants of the two pushes ---------------------------------------------------
// A push that has the GPU to itself (synchronous exchange) moves its rows with the copy unit instead of with
// the SMs' load/store pipes: one warp per CTA streams chunks of rows through a ring of shared-memory buffers
// (cp.async.bulk: global -> shared, completing on an mbarrier; shared -> global, local or peer, tracked in
// bulk async-groups).  Local and remote destinations no longer share store queues, and the requests that
// cross NVLink are whole rows.  The SIMT kernels above remain for pushes that run next to a GEMM on another
// stream (they need no shared memory and fit beside its CTAs).
constexpr int kBulkBufs = 4;
constexpr int kBulkBufBytes = 32768;
constexpr int kBulkLag = kBulkBufs - 2;  // chunks between a buffer's load and its stores
constexpr uint64_t kBulkWaitLimitNs = 1000ull * 1000ull * 1000ull;

__device__ __forceinline__ uint32_t smem_addr32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void bulk_bar_init(uint32_t bar) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all but the most recent group of this thread have finished reading shared memory
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
// every group of this thread is complete: its writes are performed
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ bool bulk_bar_wait(uint32_t bar, uint32_t parity) {
  const uint64_t t0 = timer_ns();
  uint32_t spins = 0;
  for (;;) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((++spins & 127u) == 0 && timer_ns() - t0 > kBulkWaitLimitNs) return false;
  }
}
// after the last store: writes of the copy unit are ordered before the flag this CTA may raise
__device__ __forceinline__ void bulk_drain() {
  bulk_wait_all();
  asm volatile("fence.proxy.async;" ::: "memory");
}

template <int K>
__global__ void __launch_bounds__(32)
ep_dispatch_bulk_kernel(const uint8_t* __restrict__ x, const int* __restrict__ pos, const int* __restrict__ seg_offsets,
                        const int* __restrict__ meta, PeerTable recv_bufs, PeerTable flags, unsigned int* done_counter,
                        int64_t n_tokens, uint32_t row_bytes, int tokens_per_chunk, int rank, int world, int el,
                        int capacity_rows, uint32_t seq, uint32_t* status) {
  extern __shared__ __align__(128) uint8_t bulk_bufs[];
  __shared__ __align__(8) uint64_t bars[kBulkBufs];
  __shared__ int s_first[kMaxRanks + 1];
  __shared__ int s_base[kMaxRanks];
  const int lane = threadIdx.x;
  pdl_trigger();
  if (lane == 0) {
    for (int b = 0; b < kBulkBufs; ++b) bulk_bar_init(smem_addr32(&bars[b]));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_wait();
  if (lane <= world) s_first[lane] = seg_offsets[lane * el];
  if (lane < world) s_base[lane] = meta[lane];
  __syncwarp();
  const int64_t n_chunks = (n_tokens + tokens_per_chunk - 1) / tokens_per_chunk;
  const int64_t mine = n_chunks > blockIdx.x ? (n_chunks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const uint32_t buf0 = smem_addr32(bulk_bufs);
  for (int64_t j = 0; j < mine + kBulkLag; ++j) {
    if (j < mine) {
      if (j >= kBulkBufs) bulk_wait_read_1();  // the stores that read this buffer are done with it
      __syncwarp();
      if (lane == 0) {
        const int64_t tok0 = (blockIdx.x + j * gridDim.x) * tokens_per_chunk;
        const int64_t left = n_tokens - tok0;
        const uint32_t n = static_cast<uint32_t>(left < tokens_per_chunk ? left : tokens_per_chunk);
        const int b = static_cast<int>(j % kBulkBufs);
        bulk_load(buf0 + b * kBulkBufBytes, x + tok0 * row_bytes, n * row_bytes, smem_addr32(&bars[b]));
      }
    }
    const int64_t k = j - kBulkLag;
    if (k >= 0) {
      const int b = static_cast<int>(k % kBulkBufs);
      // the same verdict in every lane, so that the warp leaves the loop together
      if (!__all_sync(0xffffffffu, bulk_bar_wait(smem_addr32(&bars[b]), static_cast<uint32_t>((k / kBulkBufs) & 1)))) {
        if (status != nullptr) atomicCAS(status, 0u, DICE_STATUS_WAIT_SMEM_FULL);
        break;
      }
      const int64_t tok0 = (blockIdx.x + k * gridDim.x) * tokens_per_chunk;
      const int64_t left = n_tokens - tok0;
      const int n = static_cast<int>(left < tokens_per_chunk ? left : tokens_per_chunk);
      if (lane < n * K) {
        const int ti = lane / K;
        const int p = pos[(tok0 + ti) * K + (lane - ti * K)];
        if (p >= 0) {
          int d = 0;
          while (d + 1 < world && p >= s_first[d + 1]) ++d;
          const int row = s_base[d] + (p - s_first[d]);
          if (row < capacity_rows)
            bulk_store(static_cast<uint8_t*>(recv_bufs.ptr[d]) + static_cast<int64_t>(row) * row_bytes,
                       buf0 + b * kBulkBufBytes + ti * row_bytes, row_bytes);
          else if (status != nullptr)
            atomicCAS(status, 0u, DICE_STATUS_EXCHANGE_OVERFLOW);
        }
      }
      bulk_commit();
    }
  }
  bulk_drain();
  signal_when_grid_done(done_counter, flags, rank, world, seq);
}

__global__ void __launch_bounds__(32)
ep_return_bulk_kernel(const uint8_t* __restrict__ rows, const int* __restrict__ meta, PeerTable back_bufs, PeerTable flags,
                      unsigned int* done_counter, uint32_t row_bytes, int rows_per_chunk, int rank, int world,
                      int back_capacity_rows, uint32_t seq, uint32_t* status) {
  extern __shared__ __align__(128) uint8_t bulk_bufs[];
  __shared__ __align__(8) uint64_t bars[kBulkBufs];
  __shared__ int s_src_off[kMaxRanks + 1];
  __shared__ int s_back[kMaxRanks];
  __shared__ int s_chunk0[kMaxRanks + 1];  // chunks before source s
  const int lane = threadIdx.x;
  pdl_trigger();
  if (lane == 0) {
    for (int b = 0; b < kBulkBufs; ++b) bulk_bar_init(smem_addr32(&bars[b]));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_wait();
  if (lane <= world) s_src_off[lane] = meta[2 * world + lane];
  if (lane < world) s_back[lane] = meta[world + lane];
  __syncwarp();
  if (lane == 0) {
    int run = 0;
    for (int s = 0; s < world; ++s) {
      s_chunk0[s] = run;
      const int n = s_src_off[s + 1] - s_src_off[s];
      run += n > 0 ? (n + rows_per_chunk - 1) / rows_per_chunk : 0;
    }
    s_chunk0[world] = run;
  }
  __syncwarp();
  const int64_t n_chunks = s_chunk0[world];
  const int64_t mine = n_chunks > blockIdx.x ? (n_chunks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const uint32_t buf0 = smem_addr32(bulk_bufs);
  // a chunk: `n` rows of source `s` starting at received row `r0`
  auto locate = [&](int64_t j, int& s, int& r0, int& n) {
    const int c = static_cast<int>(blockIdx.x + j * gridDim.x);
    s = 0;
    while (s + 1 < world && c >= s_chunk0[s + 1]) ++s;
    r0 = s_src_off[s] + (c - s_chunk0[s]) * rows_per_chunk;
    n = s_src_off[s + 1] - r0;
    if (n > rows_per_chunk) n = rows_per_chunk;
  };
  if (lane == 0) {  // the whole pipeline is one lane's: one load and one store per chunk
    bool alive = true;
    for (int64_t j = 0; alive && j < mine + kBulkLag; ++j) {
      if (j < mine) {
        if (j >= kBulkBufs) bulk_wait_read_1();
        int s, r0, n;
        locate(j, s, r0, n);
        const int b = static_cast<int>(j % kBulkBufs);
        bulk_load(buf0 + b * kBulkBufBytes, rows + static_cast<int64_t>(r0) * row_bytes, static_cast<uint32_t>(n) * row_bytes,
                  smem_addr32(&bars[b]));
      }
      const int64_t k = j - kBulkLag;
      if (k >= 0) {
        const int b = static_cast<int>(k % kBulkBufs);
        if (!bulk_bar_wait(smem_addr32(&bars[b]), static_cast<uint32_t>((k / kBulkBufs) & 1))) {
          if (status != nullptr) atomicCAS(status, 0u, DICE_STATUS_WAIT_SMEM_FULL);
          alive = false;
          break;
        }
        int s, r0, n;
        locate(k, s, r0, n);
        const int row = s_back[s] + (r0 - s_src_off[s]);
        if (row + n > back_capacity_rows) {
          if (status != nullptr) atomicCAS(status, 0u, DICE_STATUS_EXCHANGE_OVERFLOW);
          n = back_capacity_rows > row ? back_capacity_rows - row : 0;
        }
        if (n > 0)
          bulk_store(static_cast<uint8_t*>(back_bufs.ptr[s]) + static_cast<int64_t>(row) * row_bytes, buf0 + b * kBulkBufBytes,
                     static_cast<uint32_t>(n) * row_bytes);
        bulk_commit();
      }
    }
    bulk_drain();
  }
  __syncwarp();
  signal_when_grid_done(done_counter, flags, rank, world, seq);
}

// DICE_EP_P2P_BULK=0 keeps the SIMT pushes everywhere
bool bulk_pushes() {
  static int cached = -1;
  if (cached < 0) {
    const char* e = getenv("DICE_EP_P2P_BULK");
    cached = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return cached != 0;
}

int sm_count_here() {
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

template <typename Kern>
int bulk_smem_ready(Kern kernel) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBulkBufs * kBulkBufBytes) ==
                 cudaSuccess
             ? DICE_OK
             : DICE_ERR_CUDA;
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
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int el = n_experts / world;
  const size_t row_bytes = hidden * es;
  if (max_ctas == 0 && bulk_pushes() && row_bytes <= kBulkBufBytes && n_tokens > 0) {
    // the push has the GPU to itself: move the rows with the copy unit
    const int sms = sm_count_here();
    if (sms <= 0) return DICE_ERR_CUDA;
    int tpc = static_cast<int>(kBulkBufBytes / row_bytes);
    if (tpc > 32 / k) tpc = 32 / k;
    const int64_t chunks = (n_tokens + tpc - 1) / tpc;
    const dim3 grid(static_cast<unsigned>(chunks < sms ? chunks : sms));
    const uint8_t* xb = static_cast<const uint8_t*>(x);
    if (k == 2) {
      DICE_CHECK_ARG(bulk_smem_ready(ep_dispatch_bulk_kernel<2>) == DICE_OK, DICE_ERR_CUDA);
      DICE_CUDA_OK(dice_launch(ep_dispatch_bulk_kernel<2>, grid, dim3(32), kBulkBufs * kBulkBufBytes, s, xb, pos, seg_offsets,
                               meta, r, f, done_counter, n_tokens, static_cast<uint32_t>(row_bytes), tpc, rank, world, el,
                               capacity_rows, seq, status));
    } else {
      DICE_CHECK_ARG(bulk_smem_ready(ep_dispatch_bulk_kernel<1>) == DICE_OK, DICE_ERR_CUDA);
      DICE_CUDA_OK(dice_launch(ep_dispatch_bulk_kernel<1>, grid, dim3(32), kBulkBufs * kBulkBufBytes, s, xb, pos, seg_offsets,
                               meta, r, f, done_counter, n_tokens, static_cast<uint32_t>(row_bytes), tpc, rank, world, el,
                               capacity_rows, seq, status));
    }
    return DICE_OK;
  }
  int64_t blocks = (n_tokens + 7) / 8;
  if (blocks < 1) blocks = 1;  // the flags are raised even when this rank has nothing to send
  if (max_ctas > 0 && blocks > max_ctas) blocks = max_ctas;  // a small grid leaves the SMs to a concurrent GEMM
  DICE_CHECK_ARG(blocks <= 0x7fffffffLL, DICE_ERR_LIMIT);
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
  const size_t row_bytes = hidden * es;
  if (max_ctas == 0 && bulk_pushes() && row_bytes <= kBulkBufBytes && max_rows > 0) {
    const int sms = sm_count_here();
    if (sms <= 0) return DICE_ERR_CUDA;
    const int rpc = static_cast<int>(kBulkBufBytes / row_bytes);
    const int64_t chunks = (static_cast<int64_t>(max_rows) + rpc - 1) / rpc + world;
    DICE_CHECK_ARG(bulk_smem_ready(ep_return_bulk_kernel) == DICE_OK, DICE_ERR_CUDA);
    DICE_CUDA_OK(dice_launch(ep_return_bulk_kernel, dim3(static_cast<unsigned>(chunks < sms ? chunks : sms)), dim3(32),
                             kBulkBufs * kBulkBufBytes, static_cast<cudaStream_t>(stream),
                             static_cast<const uint8_t*>(rows), meta, b, f, done_counter, static_cast<uint32_t>(row_bytes), rpc,
                             rank, world, back_capacity_rows, seq, status));
    return DICE_OK;
  }
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
