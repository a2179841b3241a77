// Version / error-text entry points of the C ABI.
#include <stdlib.h>

#include <atomic>

#include "common.cuh"

static std::atomic<uint64_t> g_kernel_launches{0};
void dice_count_launch() { g_kernel_launches.fetch_add(1, std::memory_order_relaxed); }
extern "C" uint64_t dice_kernel_launches(void) { return g_kernel_launches.load(std::memory_order_relaxed); }

bool dice_pdl_enabled() {
  static int cached = -1;
  if (cached < 0) {
    const char* e = getenv("DICE_PDL");
    cached = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return cached != 0;
}

extern "C" int dice_abi_version(void) { return DICE_ABI_VERSION; }

extern "C" const char* dice_strerror(int code) {
  switch (code) {
    case DICE_OK: return "ok";
    case DICE_ERR_ARG: return "invalid argument (null pointer or negative size)";
    case DICE_ERR_SHAPE: return "unsupported shape or divisibility";
    case DICE_ERR_DTYPE: return "unsupported element type";
    case DICE_ERR_ALIGN: return "pointer is not 16-byte aligned";
    case DICE_ERR_SCRATCH: return "scratch buffer too small";
    case DICE_ERR_CUDA: return "a CUDA call failed";
    case DICE_ERR_LIMIT: return "size exceeds a documented maximum";
    default: return "unknown dice_b200 error code";
  }
}

extern "C" const char* dice_status_message(uint32_t status) {
  switch (status) {
    case DICE_STATUS_OK: return "ok";
    case DICE_STATUS_WAIT_SMEM_FULL: return "timed out waiting for operand tiles to arrive in shared memory";
    case DICE_STATUS_WAIT_SMEM_EMPTY: return "timed out waiting for a shared-memory ring slot to be released";
    case DICE_STATUS_WAIT_ACC_FULL: return "timed out waiting for an accumulator to complete";
    case DICE_STATUS_WAIT_ACC_EMPTY: return "timed out waiting for an accumulator to be drained";
    case DICE_STATUS_BAD_SEGMENTS: return "segment offsets are not monotone or exceed the row count";
    case DICE_STATUS_WAIT_PEER_COUNTS: return "timed out waiting for a peer rank's row counts";
    case DICE_STATUS_WAIT_PEER_DISPATCH: return "timed out waiting for a peer rank's dispatched rows";
    case DICE_STATUS_WAIT_PEER_COMBINE: return "timed out waiting for a peer rank's expert outputs";
    case DICE_STATUS_EXCHANGE_OVERFLOW: return "a rank received more rows than its exchange buffer holds";
    case DICE_STATUS_PEER_FAILED: return "a peer rank reported that the rows it sent are incomplete";
    case DICE_STATUS_WAIT_FFN_ROWS: return "timed out waiting for the expert outputs that a return push follows";
    default: return "unknown device status";
  }
}
