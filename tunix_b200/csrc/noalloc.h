// Allocation-free C entry point of libtunix_b200_cuda.so. It has no counterpart in the reference
// (bigdatamark/tunix has no native GPU code); it exists for callers of this library that are not
// allowed to allocate device memory.
//
// Who that is: host code that runs while cudaMalloc is illegal or unwanted -- inside a stream
// capture, inside a process whose whole device-memory budget is owned by another component (an
// inference server's pre-reserved pool, a framework allocator you must not bypass), or a bare
// C/C++ program that links this library without torch and has no allocator to lend us.
//
// What it does: flash-attention backward, same math as tb_attn_bwd, but the two scratch buffers
// that tb_attn_bwd takes from its caller (the per-row delta and the fp32 dQ accumulator) live in
// a fixed array inside the library image. Inputs and outputs are still the caller's.
//
// Limits and rules
//   * B*Tq*N*H <= TB_NOALLOC_MAX_DQ_ELEMS (4 Mi elements, 16 MiB) and B*N*Tq <= TB_NOALLOC_MAX_ROWS
//     (256 Ki rows, 1 MiB). Larger problems are rejected with -11 and a message from
//     tb_noalloc_last_error(); nothing is launched. Every GPU that loads the library carries these
//     17 MiB until the process exits, whether or not the entry point is ever called.
//   * The first call on a device looks up the scratch addresses (cudaGetSymbolAddress, with that
//     device current). Make that first call outside any stream capture.
//   * All calls on a device share the one scratch array and it keeps the previous call's contents;
//     the entry point clears the part it needs to start from zero. Two calls that overlap on the GPU
//     (different streams, no ordering between them) race on it: serialise them.
//   * No cudaMalloc / cudaFree / allocating library routine is called.
//   * Layout: q, o, dout, dq are [B*Tq, N*H] bf16 contiguous; k, v, dk, dv are [B*Tk, KH*H] bf16
//     contiguous; lse is [B, N, Tq] fp32 from the forward pass; status is a device int that receives
//     a non-zero code if a bounded wait inside the kernel gives up (may be null).
//   * No segment ids; query i sits at key position i + (Tk - Tq).
//   * Host threads: the one-time address lookup is guarded by a mutex, and tb_noalloc_last_error()
//     returns the message of the calling thread's own last call (thread-local storage). The GPU-side
//     rule above still holds: calls from different threads must not overlap on the device.
// Returns 0 on success, a negative code otherwise.
#pragma once
#include <cuda_runtime.h>

#define TB_NOALLOC_MAX_DQ_ELEMS (4 * 1024 * 1024)
#define TB_NOALLOC_MAX_ROWS (256 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int tb_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* o, const void* dout,
                        const float* lse, void* dq, void* dk, void* dv, int B, int Tq, int Tk, int N, int KH,
                        int H, float scale, float softcap, int causal, int window, int* status,
                        cudaStream_t stream);

const char* tb_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
