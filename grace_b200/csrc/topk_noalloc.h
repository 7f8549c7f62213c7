// Allocation-free top-k selection.  This entry point has no counterpart in the
// reference (whose only native top-k, radixtopk_cuda/rdxtopk_cuda.cu, calls
// cudaMalloc and cudaFree on every invocation); it exists for callers of this
// library that are not allowed to allocate device memory at the point where
// they need a top-k: code running inside a memory-planned region that has
// already handed out every byte it reserved, plug-ins loaded into a host
// process that owns the allocator and forbids foreign cudaMalloc calls, and
// latency-critical loops where an allocation would synchronise the device.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Selects the k entries of largest magnitude of x[0..n) (fp32, device memory,
// 16-byte aligned).  Writes their signed values to values[0..k) and their
// positions to indices[0..k), in no particular order; ties at the k-th
// magnitude are broken arbitrarily.  Same result set as
// grace_b200.ops.sparse.topk_select.
//
// Memory: the call allocates nothing, neither with cudaMalloc / cudaFree nor
// through any library.  Its work area (a 4096-bin histogram, the radix-select
// state, a grid-barrier word, a status word and the output counter: 16 640
// bytes, kGraceTopkNoallocScratchBytes) is a file-scope __device__ array inside
// this library, so every GPU that loads the library holds those bytes until
// the process exits.
//
// Limits: 1 <= k <= n <= 2^31 - 1 (kGraceTopkNoallocMaxElems); larger inputs
// are rejected with GRACE_NOALLOC_TOO_LARGE and nothing is launched.
//
// First call on a device: resolves the device address of the work area
// (cudaGetSymbolAddress, with that device current) and queries the launch
// geometry.  Make that first call outside of any stream capture; later calls
// only enqueue a memset of the work area and one kernel on `stream`.
//
// Sharing: all calls on a device use the same work area, which still holds
// the previous call's contents when a call begins; the call clears the parts
// that must start from zero itself.  Two calls that overlap on the GPU (issued
// on different streams without ordering, or from two host threads) race on
// that area and produce garbage: serialise them.
//
// Returns 0 when the work was enqueued, a negative GRACE_NOALLOC_* code
// otherwise.  `stream` is a cudaStream_t (0 = default stream).  Completion is
// observed through the stream as usual.  One failure is NOT a CUDA error and
// does not show on the stream: the kernel's grid-wide barriers give up after
// ten seconds (a co-resident grid that never assembles); the kernel then
// records the fact in the status words of the work area, skips the rest of its
// work and returns, leaving values / indices unwritten.  Read those words with
// grace_topk_noalloc_status() before trusting the outputs of a call whose
// latency looked wrong, or after every call if you can afford the stream
// synchronisation.
int grace_topk_select_noalloc(const float* x, long long n, int k, float* values, int* indices, void* stream);

// Copies the four status words of the work area of the CURRENT device to
// out[0..4) (host memory) after everything queued on `stream` so far has
// finished: out[0] = 0 when the last grace_topk_select_noalloc call on this
// device ran to completion, 1 when a grid barrier timed out (out[1] = index of
// that barrier).  The next grace_topk_select_noalloc call clears the words, so
// ask before issuing it.  Allocates nothing; blocks the calling thread until
// `stream` is idle.  Returns 0, or GRACE_NOALLOC_SETUP_FAILED when no call has
// set up this device yet, or GRACE_NOALLOC_LAUNCH_FAILED when the copy failed.
int grace_topk_noalloc_status(unsigned out[4], void* stream);

// Human-readable text for a return code of the function above.
const char* grace_topk_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif

#define GRACE_NOALLOC_OK 0
#define GRACE_NOALLOC_BAD_ARGUMENT (-1)   /* null pointer, k < 1, k > n, x not 16-byte aligned */
#define GRACE_NOALLOC_TOO_LARGE (-2)      /* n beyond kGraceTopkNoallocMaxElems */
#define GRACE_NOALLOC_SETUP_FAILED (-3)   /* cudaGetSymbolAddress / occupancy query failed */
#define GRACE_NOALLOC_LAUNCH_FAILED (-4)  /* memset or kernel launch was refused */

#define kGraceTopkNoallocMaxElems 2147483647LL
#define kGraceTopkNoallocScratchBytes 16640
