// Allocation-free entry point of the kernel library.  It has no counterpart in the reference engine.
//
// Some callers may not allocate device memory at the moment they need a kernel: an engine whose memory plan is fixed
// once the model is loaded, a callback running inside another framework's stream, a host thread that must not touch
// the allocator.  rx_topk_static is rx_topk for them: the scratch that rx_topk takes from its caller sits in a fixed
// 2 MiB array inside the library (held by every GPU that loads the library, until the process exits).
//
//   logits : float32 [rows, vocab] on the device, contiguous
//   ids    : int32   [rows, count] out, ordered (value descending, id ascending)
//   vals   : float32 [rows, count] out
//   limits : rows <= 64, vocab <= 262144, 1 <= count <= 64; larger sizes return cudaErrorInvalidValue (1)
//   returns 0 or a cudaError_t
//
// The first call on a device resolves the array's device address; make it before any stream capture.  All calls share
// the array: calls that overlap on the GPU race, so keep them on one stream or order them with events.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
int rx_topk_static(const void* logits, int rows, int vocab, int count, void* ids, void* vals, void* stream);
#ifdef __cplusplus
}
#endif
