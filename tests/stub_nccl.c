/*
 * A stand-in for libnccl.so.2 with one rank, for the host-side failure tests of the expert-parallel layer.
 * Test infrastructure only: the library under test binds it through NVMOE_NCCL_LIBRARY in a process that
 * has no real NCCL loaded.  A send to oneself followed by the matching receive is a device-to-device copy on
 * the caller's stream; every call is counted; a chosen send can be made to fail, and the asynchronous error
 * query can be made to report a failure, so that the error paths are reached from the host without any GPU
 * fault.
 */
#include <cuda_runtime.h>
#include <stddef.h>
#include <string.h>

typedef enum { ncclSuccess = 0, ncclUnhandledCudaError = 1, ncclSystemError = 2, ncclInternalError = 3, ncclInvalidArgument = 4,
               ncclInvalidUsage = 5, ncclRemoteError = 6, ncclInProgress = 7 } ncclResult_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef struct stub_comm { int world; int rank; int aborted; } * ncclComm_t;
typedef int ncclDataType_t;

enum { kGroupStart, kGroupEnd, kSend, kRecv, kAbort, kAsyncPoll, kDestroy, kCounters };
static int g_count[kCounters];
static int g_fail_send_in = -1;     /* the n-th send from now fails (0 = the next one); -1 = never */
static int g_async_error = 0;
static struct { const void* ptr; size_t bytes; } g_pending[64];
static int g_pending_head = 0, g_pending_tail = 0;
static struct stub_comm g_comm;

void stub_nccl_counters(int* out) { memcpy(out, g_count, sizeof g_count); }
void stub_nccl_reset(void) { memset(g_count, 0, sizeof g_count); g_fail_send_in = -1; g_async_error = 0; g_pending_head = g_pending_tail = 0; }
void stub_nccl_fail_send_in(int n) { g_fail_send_in = n; }
void stub_nccl_set_async_error(int on) { g_async_error = on; }

const char* ncclGetErrorString(ncclResult_t r) { return r == ncclSuccess ? "no error" : r == ncclInternalError ? "injected send failure" : "injected asynchronous failure"; }
ncclResult_t ncclGetUniqueId(ncclUniqueId* id) { memset(id, 7, sizeof *id); return ncclSuccess; }
ncclResult_t ncclCommInitRank(ncclComm_t* comm, int world, ncclUniqueId id, int rank) {
    (void)id;
    if (world != 1 || rank != 0) return ncclInvalidArgument;
    g_comm.world = 1; g_comm.rank = 0; g_comm.aborted = 0;
    *comm = &g_comm;
    return ncclSuccess;
}
ncclResult_t ncclCommDestroy(ncclComm_t comm) { (void)comm; g_count[kDestroy]++; return ncclSuccess; }
ncclResult_t ncclCommAbort(ncclComm_t comm) { comm->aborted = 1; g_count[kAbort]++; return ncclSuccess; }
ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* error) {
    (void)comm;
    g_count[kAsyncPoll]++;
    *error = g_async_error ? ncclSystemError : ncclSuccess;
    return ncclSuccess;
}
ncclResult_t ncclGroupStart(void) { g_count[kGroupStart]++; return ncclSuccess; }
ncclResult_t ncclGroupEnd(void) { g_count[kGroupEnd]++; g_pending_head = g_pending_tail = 0; return ncclSuccess; }
ncclResult_t ncclSend(const void* buf, size_t count, ncclDataType_t type, int peer, ncclComm_t comm, cudaStream_t stream) {
    (void)type; (void)comm; (void)stream;
    g_count[kSend]++;
    if (g_fail_send_in == 0) { g_fail_send_in = -1; return ncclInternalError; }
    if (g_fail_send_in > 0) g_fail_send_in--;
    if (peer != 0 || g_pending_tail >= 64) return ncclInvalidArgument;
    g_pending[g_pending_tail].ptr = buf;
    g_pending[g_pending_tail].bytes = count;
    g_pending_tail++;
    return ncclSuccess;
}
ncclResult_t ncclRecv(void* buf, size_t count, ncclDataType_t type, int peer, ncclComm_t comm, cudaStream_t stream) {
    (void)type; (void)comm;
    g_count[kRecv]++;
    if (peer != 0 || g_pending_head >= g_pending_tail || g_pending[g_pending_head].bytes != count) return ncclInvalidArgument;
    const void* src = g_pending[g_pending_head++].ptr;
    return cudaMemcpyAsync(buf, src, count, cudaMemcpyDeviceToDevice, stream) == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError;
}
