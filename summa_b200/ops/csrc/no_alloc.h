// Allocation-free entry point of the kernel library. It has no counterpart in the
// reference project; it exists for hosts that embed this library but do not let it
// allocate device memory.
//
// Who needs it: a serving process that hands the whole GPU to its own memory manager at
// start-up (so a later cudaMalloc from a plugin either fails or stalls the device), or an
// application that loads this .so through its C ABI only, passes in the input and output
// buffers it owns, and has no way to give the library a workspace. Such callers cannot
// provide the `delta` scratch buffer that sb_attention_bwd expects, and the Python layer
// (which gets it from the PyTorch allocator) is not available to them.
//
// sb_attention_bwd_noalloc computes exactly what sb_attention_bwd computes — dq, dk, dv of
// the flash-attention forward — but keeps its scratch in a fixed array inside the library:
//   * capacity: batch * query_heads * roundup(query_length, 64) <= 1,048,576 (two arrays of
//     that many floats: 8 MiB of device memory, held by every GPU that loads the library
//     until the process exits). Larger problems are refused with SB_ERR_TOO_LARGE (-4) and
//     a message on stderr.
//   * it calls no cudaMalloc / cudaFree and no allocating library routine; the word the
//     kernels use to report a timed-out wait is a static device word too. That word is NOT the
//     one sb_read_error_flag reads (which allocates on first use): read it with
//     sb_attention_bwd_noalloc_status after the call, and treat a non-zero value as "the
//     gradients of that call are not valid".
//   * the first call on a device looks up the device addresses of the built-in arrays
//     (cudaGetSymbolAddress, with that device current; host threads racing on the first call
//     are ordered by std::call_once). Make that first call before any stream capture begins.
//   * every call on a device shares the one array. Nothing in it has to start at zero
//     (the first kernel overwrites every value the later kernels read), but two calls that
//     overlap on the GPU — different streams, or different host threads — would race on
//     it: issue them on one stream, or otherwise order them.
// Arguments are those of sb_attention_bwd without the `delta` pointer.
#pragma once
#include <cuda_runtime.h>

extern "C" int sb_attention_bwd_noalloc(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                        const float* lse, void* dq, void* dk, void* dv, int B, int Hq, int Hkv, int Sq,
                                        int Sk, int D, const long* q_strides, const long* k_strides,
                                        const long* v_strides, const long* o_strides, const long* dout_strides,
                                        const long* dq_strides, const long* dk_strides, const long* dv_strides,
                                        int causal, int window, int q_offset, float scale, cudaStream_t stream);

// Status word of the allocation-free path on the current device: 0 = clean, bit 1 = a bounded
// mbarrier wait inside the kernels gave up (outputs of that call are garbage). Synchronises the
// device, reads the static word and clears it; allocates nothing.
extern "C" int sb_attention_bwd_noalloc_status(unsigned int* out);
