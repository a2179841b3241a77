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
//
// Failures travel with the flags.  A flag array holds 64 words: [0, W) the
// flags proper and [32, 32 + W) failure marks.  A push that could not complete
// (its count exchange timed out, or one of its copies never arrived) writes the
// exchange's sequence number into its failure mark on every peer before it
// raises the flag, so that the peers, which would otherwise consume incomplete
// rows with a clean status, record DICE_STATUS_PEER_FAILED themselves.
//
// A receive buffer that is too small for what the peers want to send is found
// by EVERY rank in the count exchange (each holds the full count matrix): all
// of them record DICE_STATUS_EXCHANGE_OVERFLOW, and the exchange degenerates to
// one that moves no rows at all (nothing is read or written out of bounds).
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace {

constexpr int kMaxRanks = 16;
constexpr int kMaxKeys = 64;  // experts
constexpr uint64_t kPeerWaitLimitNs = 2000ull * 1000ull * 1000ull;
// How long a kernel waits for another rank (a flag) or for the GEMM it follows (block counters) before it records
// the expired wait and returns: 2 s unless dice_ep_set_wait_limit_ms() changed it on this device.  Ranks that drift
// apart by more than this between two exchanges (one of them stalled on the host) fail instead of waiting.
__device__ unsigned long long g_peer_wait_limit_ns = kPeerWaitLimitNs;

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
constexpr int kFailMarkBase = 32;  // failure marks of a flag array start at this word

// meta block, fixed part (see meta_ints below)
constexpr int kMetaTotal = 0;   // rows this rank receives
constexpr int kMetaState = 1;   // 0 ok, kStateOverflow, kStateNoCounts
constexpr int kMetaHead = 2;
constexpr int kStateOverflow = 1;
constexpr int kStateNoCounts = 2;

// true when *flag reached `seq` within the time limit
__device__ bool wait_flag(const uint32_t* flag, uint32_t seq, uint32_t* status, uint32_t code) {
  const uint64_t t0 = timer_ns();
  const uint64_t limit = g_peer_wait_limit_ns;
  uint32_t spins = 0;
  for (;;) {
    if (static_cast<int32_t>(ld_acquire_sys(flag) - seq) >= 0) return true;
    if ((++spins & 63u) == 0) {
      if (timer_ns() - t0 > limit) {
        if (status != nullptr) atomicCAS(status, 0u, code);
        return false;
      }
      __nanosleep(200);
    }
  }
}

// Layout of the per-slot meta block (int32) that describes what this rank receives and where its own rows go.
// It is derived by ep_counts_kernel (packed layout) or by ep_wait_dispatch_kernel (region layout):
//   [0]                 total rows this rank receives
//   [1]                 state: 0 ok, 1 a receive buffer would overflow, 2 the peers' counts never arrived
//   send_base[W]        first row of this rank's block in peer d's dispatch buffer
//   back_base[W]        first row of this rank's block in peer s's combine buffer
//   src_off[W+1]        first row received from source s
//   src_cnt[W]          rows received from source s
//   seg_off[...]        offsets of the segments of the receive buffer, ready for the grouped GEMM:
//                       packed layout: W*El segments in (source, slot) order;
//                       region layout: W*(El+1) segments, every source's El slots followed by the unused rest
//                       of its region (weight slab -1: skipped by the GEMM)
__host__ __device__ inline int meta_ints(int w, int el) { return kMetaHead + 4 * w + 1 + w * (el + 1) + 1; }
__host__ __device__ inline int meta_seg_base(int w) { return kMetaHead + 4 * w + 1; }

// Two layouts of a receive buffer.
//  * packed: the sources' blocks follow one another without gaps; a source learns where its block starts from
//    the other sources' counts, so a count exchange (a rendezvous of all ranks) precedes the dispatch.  Works
//    for any capacity.
//  * regions (region_rows > 0): source s owns rows [s * region_rows, (s+1) * region_rows) of every receive
//    buffer, where region_rows is at least the largest number of rows any rank ever sends.  A source then
//    needs nobody's counts: the dispatch publishes this rank's counts along with its rows, and the receiver
//    derives its segment table from the count matrix after the flags are up.  No count exchange, no rendezvous,
//    and no routing can overflow; it needs capacity_rows = W * region_rows.

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
  pdl_trigger();  // only now (see ep_wait_kernel)
  for (int i = threadIdx.x; i < world * n_keys; i += blockDim.x)
    s_cnt[i / n_keys][i % n_keys] = s_ok ? my_matrix[i] : 0;
  __syncthreads();
  if (threadIdx.x == 0) {
    int* send_base = meta + kMetaHead;
    int* back_base = send_base + world;
    int* src_off = back_base + world;
    int* src_cnt = src_off + world + 1;
    int* seg_off = meta + meta_seg_base(world);
    // rows source s sends to owner d
    auto block_rows = [&](int s, int d) {
      int n = 0;
      for (int i = 0; i < el; ++i) n += s_cnt[s][d * el + i];
      return n;
    };
    // every rank sees the whole matrix, so every rank finds an overflow anywhere
    bool overflow = false;
    for (int d = 0; d < world; ++d) {
      int64_t tot = 0;
      for (int s = 0; s < world; ++s) tot += block_rows(s, d);
      overflow = overflow || tot > capacity_rows;
    }
    const int state = !s_ok ? kStateNoCounts : (overflow ? kStateOverflow : 0);
    if (state == 0) {
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
        src_cnt[s] = run - src_off[s];
      }
      src_off[world] = run;
      seg_off[seg] = run;
      meta[kMetaTotal] = run;
    } else {
      // the exchange moves nothing: every destination row lies "beyond the buffer", no rows are received,
      // no segment holds work (the layer's result is invalid and flagged on every rank)
      if (state == kStateOverflow && status != nullptr) atomicCAS(status, 0u, DICE_STATUS_EXCHANGE_OVERFLOW);
      for (int d = 0; d < world; ++d) { send_base[d] = capacity_rows; back_base[d] = 0; src_cnt[d] = 0; }
      for (int s = 0; s <= world; ++s) src_off[s] = 0;
      for (int i = 0; i <= world * el; ++i) seg_off[i] = 0;
      meta[kMetaTotal] = 0;
    }
    meta[kMetaState] = state;
  }
}

// Raise `flag[rank] = seq` on every peer once the whole grid has finished writing.  `fail` (shared memory,
// non-zero when this CTA could not complete its part) is collected over the grid in the upper half of the
// counter; the last CTA then writes the failure marks before it raises the flags.  Grids stay below 65536 CTAs.
__device__ __forceinline__ void signal_when_grid_done(unsigned int* done_counter, PeerTable flags, int rank, int world,
                                                      uint32_t seq, const int* fail, unsigned int* clear = nullptr,
                                                      int clear_ints = 0) {
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last, s_any_fail;
  if (threadIdx.x == 0) {
    const unsigned int inc = *fail != 0 ? 0x10001u : 1u;
    const unsigned int now = atomicAdd(done_counter, inc) + inc;
    s_last = (now & 0xffffu) == gridDim.x;
    s_any_fail = (now >> 16) != 0u;
  }
  __syncthreads();
  if (s_last) {
    // counters that this grid consumed (the blocks of a GEMM output it followed) start from zero next time
    for (int i = threadIdx.x; i < clear_ints; i += blockDim.x) clear[i] = 0u;
    __threadfence_system();
    if (threadIdx.x < world) {
      uint32_t* f = static_cast<uint32_t*>(flags.ptr[threadIdx.x]);
      if (s_any_fail) f[kFailMarkBase + rank] = seq;  // ordered before the flag by the release store below
      st_release_sys(f + rank, seq);
    }
    if (threadIdx.x == 0) *done_counter = 0;  // ready for the next launch on this stream
  }
}

// ---- 2. dispatch: permutation gather fused with the push into the owners' buffers --------
// What every dispatch CTA needs first: where each owner's block starts in this rank's sorted order and where this
// rank's rows start in each owner's buffer.  In the region layout the latter is fixed, and block 0 publishes this
// rank's counts in every peer's matrix (ordered before the flags by the fences of signal_when_grid_done).
__device__ __forceinline__ void dispatch_prologue(const int* __restrict__ seg_offsets, const int* __restrict__ meta,
                                                  const PeerTable& matrices, int rank, int world, int el, int region_rows,
                                                  int* s_first, int* s_base, int* s_fail) {
  if (threadIdx.x <= world) s_first[threadIdx.x] = seg_offsets[threadIdx.x * el];
  if (region_rows > 0) {
    if (threadIdx.x < world) s_base[threadIdx.x] = rank * region_rows;
    if (threadIdx.x == 0) *s_fail = 0;
    if (blockIdx.x == 0) {
      const int n_keys = world * el;
      for (int i = threadIdx.x; i < world * n_keys; i += blockDim.x) {
        const int d = i / n_keys, e = i - d * n_keys;
        static_cast<int*>(matrices.ptr[d])[rank * n_keys + e] = seg_offsets[e + 1] - seg_offsets[e];
      }
    }
  } else {
    if (threadIdx.x < world) s_base[threadIdx.x] = meta[kMetaHead + threadIdx.x];
    if (threadIdx.x == 0) *s_fail = meta[kMetaState] == kStateNoCounts;
  }
}

template <int K>
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const uint4* __restrict__ x, const int* __restrict__ pos, const int* __restrict__ seg_offsets,
                   const int* __restrict__ meta, PeerTable recv_bufs, PeerTable flags, unsigned int* done_counter,
                   int64_t n_tokens, int row_vec, int rank, int world, int el, int capacity_rows, uint32_t seq,
                   uint32_t* status, int region_rows, PeerTable matrices) {
  __shared__ int s_first[kMaxRanks + 1];  // first sorted position of each owner's block
  __shared__ int s_base[kMaxRanks];
  __shared__ int s_fail;
  pdl_trigger();
  pdl_wait();
  dispatch_prologue(seg_offsets, meta, matrices, rank, world, el, region_rows, s_first, s_base, &s_fail);
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
  signal_when_grid_done(done_counter, flags, rank, world, seq, &s_fail);
}

// ---- 3. wait for all sources ------------------------------------------------------------
__global__ void ep_wait_kernel(const uint32_t* __restrict__ my_flags, int world, uint32_t seq, uint32_t* status,
                               uint32_t code) {
  pdl_wait();
  if (threadIdx.x < world) {
    if (wait_flag(my_flags + threadIdx.x, seq, status, code) &&
        ld_acquire_sys(my_flags + kFailMarkBase + threadIdx.x) == seq && status != nullptr)
      atomicCAS(status, 0u, DICE_STATUS_PEER_FAILED);  // the source says its rows are incomplete
  }
  __syncwarp();
  // The kernels behind this one may become resident only NOW, not while it spins: their blocks, parked in
  // griddepcontrol.wait, hold shared memory and thread slots on every SM, and a push of another stream of THIS GPU
  // that the flags depend on (the return that follows the second GEMM, queued behind earlier pushes) would find no
  // SM to start on.  That cycle ended only when the bounded wait ran out.
  pdl_trigger();
}

// Region layout: wait for every source's rows, then derive the meta block from the count matrix the sources
// published with them (segments of the receive buffer for the grouped GEMM, where the outputs go back to).
__global__ void __launch_bounds__(256)
ep_wait_dispatch_kernel(const uint32_t* __restrict__ my_flags, const int* __restrict__ my_matrix, int* __restrict__ meta,
                        int rank, int world, int n_keys, int region_rows, uint32_t seq, uint32_t* status) {
  __shared__ int s_cnt[kMaxRanks][kMaxKeys];
  __shared__ int s_ok;
  const int el = n_keys / world;
  pdl_wait();
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    if (!wait_flag(my_flags + threadIdx.x, seq, status, DICE_STATUS_WAIT_PEER_DISPATCH)) {
      s_ok = 0;
    } else if (ld_acquire_sys(my_flags + kFailMarkBase + threadIdx.x) == seq) {
      if (status != nullptr) atomicCAS(status, 0u, DICE_STATUS_PEER_FAILED);
      s_ok = 0;
    }
  }
  __syncthreads();
  pdl_trigger();  // only now: nothing behind this kernel becomes resident while it spins (see ep_wait_kernel)
  for (int i = threadIdx.x; i < world * n_keys; i += blockDim.x)
    s_cnt[i / n_keys][i % n_keys] = s_ok ? my_matrix[i] : 0;
  __syncthreads();
  if (threadIdx.x == 0) {
    int* send_base = meta + kMetaHead;
    int* back_base = send_base + world;
    int* src_off = back_base + world;
    int* src_cnt = src_off + world + 1;
    int* seg_off = meta + meta_seg_base(world);
    int total = 0, seg = 0;
    for (int s = 0; s < world; ++s) {
      send_base[s] = rank * region_rows;
      int before = 0;  // rows of source s for the owners in front of this rank: where this rank's outputs go back to
      for (int d = 0; d < rank; ++d)
        for (int i = 0; i < el; ++i) before += s_cnt[s][d * el + i];
      back_base[s] = before;
      src_off[s] = s * region_rows;
      int run = s * region_rows;
      for (int i = 0; i < el; ++i) {
        seg_off[seg++] = run;
        run += s_cnt[s][rank * el + i];
      }
      // a source can never send more than its region holds; a count that says otherwise is not believed
      if (run > (s + 1) * region_rows) run = (s + 1) * region_rows;
      seg_off[seg++] = run;  // the unused rest of the region: a segment without a weight slab
      src_cnt[s] = run - s * region_rows;
      total += src_cnt[s];
    }
    src_off[world] = world * region_rows;
    seg_off[seg] = world * region_rows;
    meta[kMetaTotal] = total;
    meta[kMetaState] = s_ok ? 0 : kStateNoCounts;
  }
}

// ---- 4. return: expert outputs go back to the token owners --------------------------------
__global__ void __launch_bounds__(256)
ep_return_kernel(const uint4* __restrict__ rows, const int* __restrict__ meta, PeerTable back_bufs, PeerTable flags,
                 unsigned int* done_counter, int row_vec, int rank, int world, int back_capacity_rows, int max_rows,
                 uint32_t seq, uint32_t* status) {
  __shared__ int s_src_off[kMaxRanks];   // first received row of source s
  __shared__ int s_pre[kMaxRanks + 1];   // rows received from the sources in front of s
  __shared__ int s_back[kMaxRanks];
  __shared__ int s_fail;
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x < world) {
    s_src_off[threadIdx.x] = meta[kMetaHead + 2 * world + threadIdx.x];
    s_back[threadIdx.x] = meta[kMetaHead + world + threadIdx.x];
  }
  if (threadIdx.x == 0) {
    s_fail = meta[kMetaState] == kStateNoCounts;
    int run = 0;
    for (int s = 0; s < world; ++s) {
      s_pre[s] = run;
      int off = meta[kMetaHead + 2 * world + s], n = meta[kMetaHead + 3 * world + 1 + s];
      if (off + n > max_rows) n = max_rows > off ? max_rows - off : 0;  // never read past the receive buffer
      run += n > 0 ? n : 0;
    }
    s_pre[world] = run;
  }
  __syncthreads();
  const int total = s_pre[world];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int64_t r = static_cast<int64_t>(blockIdx.x) * 8 + warp; r < total; r += static_cast<int64_t>(gridDim.x) * 8) {
    int s = 0;
    while (s + 1 < world && r >= s_pre[s + 1]) ++s;
    const int j = static_cast<int>(r - s_pre[s]);
    const int row = s_back[s] + j;
    if (row >= back_capacity_rows) {
      if (lane == 0 && status != nullptr) atomicCAS(status, 0u, DICE_STATUS_EXCHANGE_OVERFLOW);
      continue;
    }
    uint4* dst = static_cast<uint4*>(back_bufs.ptr[s]) + static_cast<int64_t>(row) * row_vec;
    const uint4* src = rows + static_cast<int64_t>(s_src_off[s] + j) * row_vec;
#pragma unroll 4
    for (int c = lane; c < row_vec; c += 32) dst[c] = ldg_stream16(src + c);
  }
  signal_when_grid_done(done_counter, flags, rank, world, seq, &s_fail);
}


// ---- bulk-copy variants of the two pushes ---------------------------------------------------
// The rows move with the copy unit instead of with the SMs' load/store pipes: a warp streams chunks of rows
// through its own ring of shared-memory buffers (cp.async.bulk: global -> shared, completing on an mbarrier;
// shared -> global, local or peer, tracked in bulk async-groups).  Local and remote destinations do not share
// store queues, and the requests that cross NVLink are whole rows.  Two shapes of the same kernels:
//   * the push has the GPU to itself (synchronous exchange): one warp per CTA, one CTA per SM, 4 x 32 KB;
//   * the push runs on a side stream next to the expert FFN (displaced / interweaved exchange): a handful of
//     CTAs of four warps with 3 x 16 KB each, launched as clusters of two so that they fill whole SM pairs;
//     the grouped GEMM leaves that many SMs free, and neither kernel disturbs the other's SMs.
// The SIMT kernels above remain as the form that needs no shared memory.
constexpr int kBulkMaxWarps = 4;
constexpr int kBulkMaxBufs = 4;
constexpr uint64_t kBulkWaitLimitNs = 1000ull * 1000ull * 1000ull;
constexpr uint64_t kBulkDrainLimitNs = 50ull * 1000ull * 1000ull;

struct BulkShape {
  int warps;           // warps per CTA, each with its own ring
  int bufs;            // buffers per ring; a buffer is stored (bufs - 2) chunks after its load was issued
  uint32_t buf_bytes;  // multiple of 128
};
__host__ __device__ inline size_t bulk_smem_bytes(const BulkShape& b) {
  return static_cast<size_t>(b.warps) * b.bufs * b.buf_bytes;
}

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
__device__ bool bulk_bar_wait(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
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
    if ((++spins & 127u) == 0 && timer_ns() - t0 > limit_ns) return false;
  }
}
// after the last store: writes of the copy unit are ordered before the flag this CTA may raise
__device__ __forceinline__ void bulk_drain() {
  bulk_wait_all();
  asm volatile("fence.proxy.async;" ::: "memory");
}
// A ring that gave up at chunk `k` still has the loads of chunks (k, last_loaded] in flight: give them a
// short, bounded time to land before the CTA's shared memory is released.
__device__ __forceinline__ void bulk_settle(const uint64_t* bars, int bufs, int64_t k, int64_t last_loaded) {
  for (int64_t i = k + 1 > 0 ? k + 1 : 0; i <= last_loaded; ++i)
    bulk_bar_wait(smem_addr32(&bars[i % bufs]), static_cast<uint32_t>((i / bufs) & 1), kBulkDrainLimitNs);
}

template <int K>
__global__ void __launch_bounds__(32 * kBulkMaxWarps)
ep_dispatch_bulk_kernel(const uint8_t* __restrict__ x, const int* __restrict__ pos, const int* __restrict__ seg_offsets,
                        const int* __restrict__ meta, PeerTable recv_bufs, PeerTable flags, unsigned int* done_counter,
                        int64_t n_tokens, uint32_t row_bytes, int tokens_per_chunk, int rank, int world, int el,
                        int capacity_rows, uint32_t seq, uint32_t* status, BulkShape shape, int region_rows,
                        PeerTable matrices) {
  extern __shared__ __align__(128) uint8_t bulk_bufs[];
  __shared__ __align__(8) uint64_t bars_all[kBulkMaxWarps][kBulkMaxBufs];
  __shared__ int s_first[kMaxRanks + 1];
  __shared__ int s_base[kMaxRanks];
  __shared__ int s_fail;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bufs = shape.bufs, lag = shape.bufs - 2;
  uint64_t* bars = bars_all[warp];
  pdl_trigger();
  if (lane == 0) {
    for (int b = 0; b < bufs; ++b) bulk_bar_init(smem_addr32(&bars[b]));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_wait();
  dispatch_prologue(seg_offsets, meta, matrices, rank, world, el, region_rows, s_first, s_base, &s_fail);
  __syncthreads();
  // every warp of the grid is one worker; chunks are dealt round-robin over the workers
  const int64_t worker = static_cast<int64_t>(blockIdx.x) * shape.warps + warp;
  const int64_t n_workers = static_cast<int64_t>(gridDim.x) * shape.warps;
  const int64_t n_chunks = (n_tokens + tokens_per_chunk - 1) / tokens_per_chunk;
  const int64_t mine = n_chunks > worker ? (n_chunks - worker + n_workers - 1) / n_workers : 0;
  const uint32_t buf0 = smem_addr32(bulk_bufs) + static_cast<uint32_t>(warp) * bufs * shape.buf_bytes;
  for (int64_t j = 0; j < mine + lag; ++j) {
    if (j < mine) {
      if (j >= bufs) bulk_wait_read_1();  // the stores that read this buffer are done with it
      __syncwarp();
      if (lane == 0) {
        const int64_t tok0 = (worker + j * n_workers) * tokens_per_chunk;
        const int64_t left = n_tokens - tok0;
        const uint32_t n = static_cast<uint32_t>(left < tokens_per_chunk ? left : tokens_per_chunk);
        const int b = static_cast<int>(j % bufs);
        bulk_load(buf0 + b * shape.buf_bytes, x + tok0 * row_bytes, n * row_bytes, smem_addr32(&bars[b]));
      }
    }
    const int64_t k = j - lag;
    if (k >= 0) {
      const int b = static_cast<int>(k % bufs);
      // the same decision in every lane, so that the warp leaves the loop together
      if (!__all_sync(0xffffffffu, bulk_bar_wait(smem_addr32(&bars[b]), static_cast<uint32_t>((k / bufs) & 1), kBulkWaitLimitNs))) {
        if (status != nullptr) atomicCAS(status, 0u, DICE_STATUS_WAIT_SMEM_FULL);
        if (lane == 0) {
          atomicExch(&s_fail, 1);
          bulk_settle(bars, bufs, k, (j < mine ? j : mine - 1));
        }
        __syncwarp();
        break;
      }
      const int64_t tok0 = (worker + k * n_workers) * tokens_per_chunk;
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
                       buf0 + b * shape.buf_bytes + ti * row_bytes, row_bytes);
          else if (status != nullptr)
            atomicCAS(status, 0u, DICE_STATUS_EXCHANGE_OVERFLOW);
        }
      }
      bulk_commit();
    }
  }
  bulk_drain();
  signal_when_grid_done(done_counter, flags, rank, world, seq, &s_fail);
}

#ifdef DICE_FOLLOW_TRACE
// debug build only: per launch of the bulk return: first start, first chunk ready (min); half, last ready, done (max)
__device__ unsigned long long g_push_trace[1024][8];
static int g_push_next = 0;
static int g_push_kind[1024];
#endif
// What a return push needs to FOLLOW a running second GEMM: the GEMM counts, per 256-row block of its tile list, the
// epilogue warps that have stored a tile (rows_done); a block is complete at `target`.  The push derives the same
// block numbering from the segment table, waits (bounded) for the blocks up to the one a chunk of rows ends in, and
// only then copies the chunk; when the grid is done its last CTA clears the counters for the next use.
struct FollowSpec {
#ifdef DICE_FOLLOW_TRACE
  int trace_id;
#endif
  unsigned int* rows_done;  // null: the rows are complete when the kernel starts
  unsigned int target;
  int n_ints;               // entries of rows_done
  const int* seg_slab;
  int n_seg;
};
constexpr int kMaxFollowSeg = 288;
constexpr int kFollowRowsPerBlock = 256;  // rows per tile pair of the CTA-pair GEMM

__global__ void __launch_bounds__(32 * kBulkMaxWarps)
ep_return_bulk_kernel(const uint8_t* __restrict__ rows, const int* __restrict__ meta, PeerTable back_bufs, PeerTable flags,
                      unsigned int* done_counter, uint32_t row_bytes, int rows_per_chunk, int rank, int world,
                      int back_capacity_rows, int max_rows, uint32_t seq, uint32_t* status, BulkShape shape,
                      FollowSpec follow) {
  __shared__ int s_fseg[kMaxFollowSeg + 1];  // segment offsets of the receive buffer
  __shared__ int s_fmb[kMaxFollowSeg + 1];   // 256-row blocks in front of segment g (-1 in the table: no weights)
  __shared__ int s_fnblk;                    // blocks of the whole output
  extern __shared__ __align__(128) uint8_t bulk_bufs[];
  __shared__ __align__(8) uint64_t bars_all[kBulkMaxWarps][kBulkMaxBufs];
  __shared__ int s_src_off[kMaxRanks];
  __shared__ int s_src_cnt[kMaxRanks];
  __shared__ int s_back[kMaxRanks];
  __shared__ int s_chunk0[kMaxRanks + 1];  // chunks before source s
  __shared__ int s_fail;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bufs = shape.bufs, lag = shape.bufs - 2;
  uint64_t* bars = bars_all[warp];
  pdl_trigger();
  if (lane == 0) {
    for (int b = 0; b < bufs; ++b) bulk_bar_init(smem_addr32(&bars[b]));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_wait();
  if (threadIdx.x < world) {
    int off = meta[kMetaHead + 2 * world + threadIdx.x], n = meta[kMetaHead + 3 * world + 1 + threadIdx.x];
    if (off + n > max_rows) n = max_rows > off ? max_rows - off : 0;  // never read past the receive buffer
    s_src_off[threadIdx.x] = off;
    s_src_cnt[threadIdx.x] = n > 0 ? n : 0;
    s_back[threadIdx.x] = meta[kMetaHead + world + threadIdx.x];
  }
  if (threadIdx.x == 0) s_fail = meta[kMetaState] == kStateNoCounts;
  if (follow.rows_done != nullptr) {
    const int* seg_off = meta + meta_seg_base(world);
    for (int g = threadIdx.x; g <= follow.n_seg; g += blockDim.x) s_fseg[g] = seg_off[g];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int s = 0; s < world; ++s) {
      s_chunk0[s] = run;
      run += (s_src_cnt[s] + rows_per_chunk - 1) / rows_per_chunk;
    }
    s_chunk0[world] = run;
    if (follow.rows_done != nullptr) {  // the GEMM's numbering of 256-row blocks (grouped_gemm_pair.cu)
      int mb = 0;
      for (int g = 0; g < follow.n_seg; ++g) {
        const int cnt = s_fseg[g + 1] - s_fseg[g];
        const bool has_weights = follow.seg_slab == nullptr || follow.seg_slab[g] >= 0;
        s_fmb[g] = has_weights ? mb : -1;
        if (cnt > 0 && has_weights) mb += (cnt + kFollowRowsPerBlock - 1) / kFollowRowsPerBlock;
      }
      s_fnblk = mb;
    }
  }
  __syncthreads();
  // Rows [.., r_last] of source s are final once every block of the GEMM's output up to the one r_last lies in
  // is complete.  The warp keeps a watermark (blocks [0, ready_upto) are complete: the GEMM finishes its blocks
  // roughly in order) and moves it with one acquire load per lane, 32 blocks per round trip.
  const bool following = follow.rows_done != nullptr;
  const int segs_per_source = following ? follow.n_seg / world : 0;
  int ready_upto = 0;
  auto last_block = [&](int s, int r_last) -> int {
    int need = -1;
    for (int g = s * segs_per_source; g < (s + 1) * segs_per_source; ++g)
      if (s_fmb[g] >= 0 && r_last >= s_fseg[g] && r_last < s_fseg[g + 1])
        need = s_fmb[g] + (r_last - s_fseg[g]) / kFollowRowsPerBlock;
    return need;
  };
  auto wait_for_block = [&](int need) -> bool {  // all lanes of the warp
    if (need >= s_fnblk || need >= follow.n_ints) return false;
    const uint64_t t0 = timer_ns();
    const uint64_t limit = g_peer_wait_limit_ns;
    uint32_t spins = 0;
    while (ready_upto <= need) {
      const int b = ready_upto + lane;
      bool done = false;
      if (b < s_fnblk) {
        unsigned int v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(follow.rows_done + b) : "memory");
        done = v >= follow.target;
      }
      const unsigned m = __ballot_sync(0xffffffffu, done);
      const int run = m == 0xffffffffu ? 32 : __ffs(static_cast<int>(~m)) - 1;
      ready_upto += run;
      if (run == 0) {
        if ((++spins & 15u) == 0) {  // lane 0's clock decides for the warp
          const int expired = timer_ns() - t0 > limit ? 1 : 0;
          if (__shfl_sync(0xffffffffu, expired, 0) != 0) return false;
        }
        __nanosleep(200);
      }
    }
    return true;
  };
#ifdef DICE_FOLLOW_TRACE
  unsigned long long* trace = g_push_trace[follow.trace_id & 1023];
  if (lane == 0) atomicMin(trace + 0, timer_ns());
#endif
  const int64_t worker = static_cast<int64_t>(blockIdx.x) * shape.warps + warp;
  const int64_t n_workers = static_cast<int64_t>(gridDim.x) * shape.warps;
  const int64_t n_chunks = s_chunk0[world];
  const int64_t mine = n_chunks > worker ? (n_chunks - worker + n_workers - 1) / n_workers : 0;
  const uint32_t buf0 = smem_addr32(bulk_bufs) + static_cast<uint32_t>(warp) * bufs * shape.buf_bytes;
  // a chunk: `n` rows of source `s` starting at received row `r0`
  auto locate = [&](int64_t j, int& s, int& r0, int& n) {
    const int c = static_cast<int>(worker + j * n_workers);
    s = 0;
    while (s + 1 < world && c >= s_chunk0[s + 1]) ++s;
    r0 = s_src_off[s] + (c - s_chunk0[s]) * rows_per_chunk;
    n = s_src_off[s] + s_src_cnt[s] - r0;
    if (n > rows_per_chunk) n = rows_per_chunk;
  };
  // A ring is one lane's: one load and one store per chunk.  A push that follows a GEMM runs the loop with the
  // whole warp (the other lanes only help to watch the block counters); every branch below is then warp-uniform.
  if (lane == 0 || following) {
    for (int64_t j = 0; j < mine + lag; ++j) {
      if (j < mine) {
        if (lane == 0 && j >= bufs) bulk_wait_read_1();
        int s, r0, n;
        locate(j, s, r0, n);
        if (following) {
          const int need = last_block(s, r0 + n - 1);
          bool ok = need < 0 || need < ready_upto || wait_for_block(need);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) {
            if (lane == 0) {
              if (status != nullptr) atomicCAS(status, 0u, DICE_STATUS_WAIT_FFN_ROWS);
              atomicExch(&s_fail, 1);
              bulk_settle(bars, bufs, j - lag - 1, j - 1);
            }
            break;
          }
          if (lane == 0) asm volatile("fence.proxy.async;" ::: "memory");  // the copy unit reads the GEMM's stores
#ifdef DICE_FOLLOW_TRACE
          if (lane == 0) {
            if (j == 0) atomicMin(trace + 1, timer_ns());
            if (j == mine / 2) atomicMax(trace + 2, timer_ns());
            if (j == mine - 1) atomicMax(trace + 3, timer_ns());
          }
#endif
        }
        if (lane == 0) {
          const int b = static_cast<int>(j % bufs);
          bulk_load(buf0 + b * shape.buf_bytes, rows + static_cast<int64_t>(r0) * row_bytes,
                    static_cast<uint32_t>(n) * row_bytes, smem_addr32(&bars[b]));
        }
      }
      const int64_t k = j - lag;
      if (k >= 0) {
        const int b = static_cast<int>(k % bufs);
        bool arrived = true;
        if (lane == 0)
          arrived = bulk_bar_wait(smem_addr32(&bars[b]), static_cast<uint32_t>((k / bufs) & 1), kBulkWaitLimitNs);
        if (following) arrived = __shfl_sync(0xffffffffu, arrived ? 1 : 0, 0) != 0;
        if (!arrived) {
          if (lane == 0) {
            if (status != nullptr) atomicCAS(status, 0u, DICE_STATUS_WAIT_SMEM_FULL);
            atomicExch(&s_fail, 1);
            bulk_settle(bars, bufs, k, (j < mine ? j : mine - 1));
          }
          break;
        }
        if (lane == 0) {
          int s, r0, n;
          locate(k, s, r0, n);
          const int row = s_back[s] + (r0 - s_src_off[s]);
          if (row + n > back_capacity_rows) {
            if (status != nullptr) atomicCAS(status, 0u, DICE_STATUS_EXCHANGE_OVERFLOW);
            n = back_capacity_rows > row ? back_capacity_rows - row : 0;
          }
          if (n > 0)
            bulk_store(static_cast<uint8_t*>(back_bufs.ptr[s]) + static_cast<int64_t>(row) * row_bytes,
                       buf0 + b * shape.buf_bytes, static_cast<uint32_t>(n) * row_bytes);
          bulk_commit();
        }
      }
    }
    if (lane == 0) bulk_drain();
#ifdef DICE_FOLLOW_TRACE
    if (lane == 0) atomicMax(trace + 4, timer_ns());
#endif
  }
  __syncwarp();
  signal_when_grid_done(done_counter, flags, rank, world, seq, &s_fail, follow.rows_done, follow.n_ints);
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

// the two shapes of the bulk-copy pushes (see above)
constexpr BulkShape kBulkAlone = {1, 4, 32768};
constexpr BulkShape kBulkBeside = {4, 3, 16384};
// (Measured on two GPUs, 18.9 MB to the peer: ring shapes of 1-8 warps x 3-4 buffers x 8-32 KB all give the same
// rates: about 495 GB/s from all SMs and 300 GB/s from 8 CTAs, against 630 GB/s for a copy-engine transfer of the
// same bytes; the limit is how fast one SM's copy unit feeds NVLink, not the depth of the rings.)

template <typename Kern>
int bulk_smem_ready(Kern kernel) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(bulk_smem_bytes(kBulkBeside) > bulk_smem_bytes(kBulkAlone)
                                                   ? bulk_smem_bytes(kBulkBeside)
                                                   : bulk_smem_bytes(kBulkAlone))) == cudaSuccess
             ? DICE_OK
             : DICE_ERR_CUDA;
}

// Launch of a push.  The form that owns the GPU is a dependent launch like the other kernels of the block.  The
// form that runs beside the expert FFN is launched as clusters of two CTAs (which fill whole SM pairs) and in
// plain stream order: with a dependent launch the next push of the side stream would become resident on a second
// set of SMs while this one still runs, and the FFN's persistent CTAs would find fewer SMs than they were sized for.
template <typename... KArgs, typename... Args>
cudaError_t launch_push(void (*kernel)(KArgs...), unsigned grid, unsigned threads, size_t smem, cudaStream_t stream,
                        bool pairs, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(threads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (pairs) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 2;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (dice_pdl_enabled() && !pairs) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  dice_count_launch();
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Grid and shape of a bulk-copy push.  max_ctas == 0: one single-warp CTA per SM; max_ctas > 0: at most that
// many four-warp CTAs, an even number of them (they are launched as clusters of two).
struct BulkPlan {
  BulkShape shape;
  unsigned grid;
  bool pairs;
};
BulkPlan plan_bulk(int max_ctas, int sms, int64_t chunks_alone, int64_t chunks_beside) {
  BulkPlan p;
  if (max_ctas == 0) {
    p.shape = kBulkAlone;
    p.grid = static_cast<unsigned>(chunks_alone < sms ? (chunks_alone > 0 ? chunks_alone : 1) : sms);
    p.pairs = false;
  } else {
    p.shape = kBulkBeside;
    int64_t ctas = (chunks_beside + p.shape.warps - 1) / p.shape.warps;
    if (ctas > max_ctas) ctas = max_ctas;
    if (ctas > sms) ctas = sms;
    ctas = (ctas + 1) & ~int64_t(1);
    if (ctas < 2) ctas = 2;
    p.grid = static_cast<unsigned>(ctas);
    p.pairs = true;
  }
  return p;
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
                                     int region_rows, const void* const* peer_matrices, uint32_t* status,
                                     void* stream) {
  DICE_CHECK_ARG(n_tokens >= 0 && hidden > 0 && done_counter && seg_offsets && region_rows >= 0, DICE_ERR_ARG);
  DICE_CHECK_ARG(region_rows > 0 || meta != nullptr, DICE_ERR_ARG);
  DICE_CHECK_ARG(region_rows == 0 || (n_experts <= kMaxKeys && static_cast<int64_t>(world) * region_rows <= capacity_rows &&
                                      n_tokens * k <= region_rows),
                 DICE_ERR_SHAPE);
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
  PeerTable m = {};
  if (region_rows > 0) {
    rc = fill_table(&m, peer_matrices, world);
    if (rc != DICE_OK) return rc;
  }
  const int row_vec = static_cast<int>(hidden * es / 16);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int el = n_experts / world;
  const size_t row_bytes = hidden * es;
  const int sms = sm_count_here();
  if (sms <= 0) return DICE_ERR_CUDA;
  if (max_ctas >= 0 && bulk_pushes() && row_bytes <= kBulkBeside.buf_bytes && n_tokens > 0) {
    auto tokens_per_chunk = [&](const BulkShape& b) {
      int t = static_cast<int>(b.buf_bytes / row_bytes);
      return t > 32 / k ? 32 / k : t;
    };
    const int tpc_alone = tokens_per_chunk(kBulkAlone), tpc_beside = tokens_per_chunk(kBulkBeside);
    const BulkPlan bp = plan_bulk(max_ctas, sms, (n_tokens + tpc_alone - 1) / tpc_alone, (n_tokens + tpc_beside - 1) / tpc_beside);
    const int tpc = max_ctas == 0 ? tpc_alone : tpc_beside;
    const uint8_t* xb = static_cast<const uint8_t*>(x);
    if (k == 2) {
      DICE_CHECK_ARG(bulk_smem_ready(ep_dispatch_bulk_kernel<2>) == DICE_OK, DICE_ERR_CUDA);
      DICE_CUDA_OK(launch_push(ep_dispatch_bulk_kernel<2>, bp.grid, 32u * bp.shape.warps, bulk_smem_bytes(bp.shape), s, bp.pairs,
                               xb, pos, seg_offsets, meta, r, f, done_counter, n_tokens, static_cast<uint32_t>(row_bytes), tpc,
                               rank, world, el, capacity_rows, seq, status, bp.shape, region_rows, m));
    } else {
      DICE_CHECK_ARG(bulk_smem_ready(ep_dispatch_bulk_kernel<1>) == DICE_OK, DICE_ERR_CUDA);
      DICE_CUDA_OK(launch_push(ep_dispatch_bulk_kernel<1>, bp.grid, 32u * bp.shape.warps, bulk_smem_bytes(bp.shape), s, bp.pairs,
                               xb, pos, seg_offsets, meta, r, f, done_counter, n_tokens, static_cast<uint32_t>(row_bytes), tpc,
                               rank, world, el, capacity_rows, seq, status, bp.shape, region_rows, m));
    }
    return DICE_OK;
  }
  int64_t blocks = (n_tokens + 7) / 8;
  if (blocks < 1) blocks = 1;  // the flags are raised even when this rank has nothing to send
  if (blocks > sms * 16) blocks = sms * 16;  // the kernel strides over the tokens
  if (max_ctas < -1 && blocks > -max_ctas) blocks = -max_ctas;
  const dim3 grid(static_cast<unsigned>(blocks));
  if (k == 2)
    DICE_CUDA_OK(dice_launch(ep_dispatch_kernel<2>, grid, dim3(256), 0, s, static_cast<const uint4*>(x), pos, seg_offsets,
                             meta, r, f, done_counter, n_tokens, row_vec, rank, world, el, capacity_rows, seq, status,
                             region_rows, m));
  else
    DICE_CUDA_OK(dice_launch(ep_dispatch_kernel<1>, grid, dim3(256), 0, s, static_cast<const uint4*>(x), pos, seg_offsets,
                             meta, r, f, done_counter, n_tokens, row_vec, rank, world, el, capacity_rows, seq, status,
                             region_rows, m));
  return DICE_OK;
}

extern "C" int dice_ep_wait_flags(const uint32_t* my_flags, int world, uint32_t seq, int what, uint32_t* status,
                                  void* stream) {
  DICE_CHECK_ARG(my_flags && world >= 1 && world <= kMaxRanks, DICE_ERR_ARG);
  const uint32_t code = (what & 1) == 0 ? DICE_STATUS_WAIT_PEER_DISPATCH : DICE_STATUS_WAIT_PEER_COMBINE;
  if ((what & 2) != 0)
    DICE_CUDA_OK(dice_launch_ordered(ep_wait_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), my_flags,
                                     world, seq, status, code));
  else
    DICE_CUDA_OK(dice_launch(ep_wait_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), my_flags, world, seq,
                             status, code));
  return DICE_OK;
}

extern "C" int dice_ep_wait_dispatch(const uint32_t* my_flags, const int32_t* my_matrix, int32_t* meta, int rank, int world,
                                     int n_experts, int region_rows, uint32_t seq, uint32_t* status, void* stream) {
  DICE_CHECK_ARG(my_flags && my_matrix && meta && world >= 1 && rank >= 0 && rank < world && region_rows > 0, DICE_ERR_ARG);
  DICE_CHECK_ARG(world <= kMaxRanks && n_experts <= kMaxKeys && n_experts % world == 0, DICE_ERR_SHAPE);
  DICE_CUDA_OK(dice_launch(ep_wait_dispatch_kernel, dim3(1), dim3(256), 0, static_cast<cudaStream_t>(stream), my_flags,
                           my_matrix, meta, rank, world, n_experts, region_rows, seq, status));
  return DICE_OK;
}

namespace {
int return_rows(const void* rows, const int32_t* meta, const void* const* peer_back, const void* const* peer_flags,
                uint32_t* done_counter, int hidden, int dtype, int rank, int world, int back_capacity_rows, int max_rows,
                uint32_t seq, int max_ctas, uint32_t* status, void* stream, const FollowSpec& follow) {
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
  const int sms = sm_count_here();
  if (sms <= 0) return DICE_ERR_CUDA;
  if (max_ctas >= 0 && bulk_pushes() && row_bytes <= kBulkBeside.buf_bytes && max_rows > 0) {
    const int rpc_alone = static_cast<int>(kBulkAlone.buf_bytes / row_bytes);
    const int rpc_beside = static_cast<int>(kBulkBeside.buf_bytes / row_bytes);
    const BulkPlan bp = plan_bulk(max_ctas, sms, (static_cast<int64_t>(max_rows) + rpc_alone - 1) / rpc_alone + world,
                                  (static_cast<int64_t>(max_rows) + rpc_beside - 1) / rpc_beside + world);
    DICE_CHECK_ARG(bulk_smem_ready(ep_return_bulk_kernel) == DICE_OK, DICE_ERR_CUDA);
    DICE_CUDA_OK(launch_push(ep_return_bulk_kernel, bp.grid, 32u * bp.shape.warps, bulk_smem_bytes(bp.shape),
                             static_cast<cudaStream_t>(stream), bp.pairs, static_cast<const uint8_t*>(rows), meta, b, f,
                             done_counter, static_cast<uint32_t>(row_bytes), max_ctas == 0 ? rpc_alone : rpc_beside, rank, world,
                             back_capacity_rows, max_rows, seq, status, bp.shape, follow));
    return DICE_OK;
  }
  DICE_CHECK_ARG(follow.rows_done == nullptr, DICE_ERR_SHAPE);  // only the bulk-copy push can follow a GEMM
  int64_t blocks = (static_cast<int64_t>(max_rows) + 7) / 8;
  if (blocks < 1) blocks = 1;
  if (blocks > sms * 16) blocks = sms * 16;  // grid-stride over the rows actually received
  if (max_ctas < -1 && blocks > -max_ctas) blocks = -max_ctas;
  DICE_CUDA_OK(dice_launch(ep_return_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0,
                           static_cast<cudaStream_t>(stream), static_cast<const uint4*>(rows), meta, b, f, done_counter,
                           row_vec, rank, world, back_capacity_rows, max_rows, seq, status));
  return DICE_OK;
}
}  // namespace

extern "C" int dice_ep_return_rows(const void* rows, const int32_t* meta, const void* const* peer_back,
                                   const void* const* peer_flags, uint32_t* done_counter, int hidden, int dtype,
                                   int rank, int world, int back_capacity_rows, int max_rows, uint32_t seq,
                                   int max_ctas, uint32_t* status, void* stream) {
#ifdef DICE_FOLLOW_TRACE
  g_push_kind[g_push_next & 1023] = max_ctas;
  const FollowSpec none = {g_push_next++, nullptr, 0u, 0, nullptr, 0};
#else
  const FollowSpec none = {nullptr, 0u, 0, nullptr, 0};
#endif
  return return_rows(rows, meta, peer_back, peer_flags, done_counter, hidden, dtype, rank, world, back_capacity_rows,
                     max_rows, seq, max_ctas, status, stream, none);
}

extern "C" int dice_ep_return_rows_following(const void* rows, const int32_t* meta, const void* const* peer_back,
                                             const void* const* peer_flags, uint32_t* done_counter, int hidden,
                                             int rank, int world, int back_capacity_rows, int max_rows, uint32_t seq,
                                             int max_ctas, uint32_t* rows_done, int rows_done_ints,
                                             const int32_t* seg_slab, int n_seg, uint32_t* status, void* stream) {
  DICE_CHECK_ARG(rows_done && rows_done_ints > 0 && max_ctas > 0 && max_rows > 0, DICE_ERR_ARG);
  DICE_CHECK_ARG(n_seg > 0 && n_seg <= kMaxFollowSeg && world >= 1 && n_seg % world == 0, DICE_ERR_LIMIT);
  // every 256-row block of the GEMM's output takes part in ceil(hidden / 256) tiles
#ifdef DICE_FOLLOW_TRACE
  g_push_kind[g_push_next & 1023] = 1000 + max_ctas;
  const FollowSpec follow = {g_push_next++, rows_done, static_cast<unsigned int>(kRowsDonePerTile * ((hidden + 255) / 256)),
                             rows_done_ints, seg_slab, n_seg};
#else
  const FollowSpec follow = {rows_done, static_cast<unsigned int>(kRowsDonePerTile * ((hidden + 255) / 256)),
                             rows_done_ints, seg_slab, n_seg};
#endif
  return return_rows(rows, meta, peer_back, peer_flags, done_counter, hidden, DICE_BF16, rank, world,
                     back_capacity_rows, max_rows, seq, max_ctas, status, stream, follow);
}

#ifdef DICE_FOLLOW_TRACE
extern "C" __attribute__((visibility("default"))) int dice_debug_push_trace(unsigned long long* out, int* kind) {
  cudaDeviceSynchronize();
  const int n = g_push_next < 1024 ? g_push_next : 1024;
  if (out != nullptr) {
    cudaMemcpyFromSymbol(out, g_push_trace, sizeof(unsigned long long) * 1024 * 8);
    for (int i = 0; i < 1024; ++i) kind[i] = g_push_kind[i];
  }
  void* pt;
  cudaGetSymbolAddress(&pt, g_push_trace);
  unsigned long long init[8] = {~0ull, ~0ull, 0, 0, 0, 0, 0, 0};
  for (int i = 0; i < 1024; ++i) cudaMemcpy(static_cast<unsigned long long*>(pt) + i * 8, init, sizeof(init), cudaMemcpyHostToDevice);
  g_push_next = 0;
  return n;
}
#endif

extern "C" int dice_ep_set_wait_limit_ms(int milliseconds) {
  DICE_CHECK_ARG(milliseconds >= 100 && milliseconds <= 3600 * 1000, DICE_ERR_ARG);
  const unsigned long long ns = static_cast<unsigned long long>(milliseconds) * 1000ull * 1000ull;
  DICE_CUDA_OK(cudaMemcpyToSymbol(g_peer_wait_limit_ns, &ns, sizeof(ns)));  // the current device's copy
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
