/* Greedy token selection for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference (taurs-ai/tau.rs always allocates its
 * argmax workspace, crates/engine/src/generation/greedy.rs:75-82); it is an addition of this
 * library.
 *
 * Who needs it: code that holds a CUDA context but may not call cudaMalloc or cudaFree where it
 * runs: a plug-in inside a host program that owns all device memory and hands out only input and
 * output buffers, a real-time loop that must not take the allocator's locks, or code that runs
 * while another part of the process is capturing a stream (an allocation there can fail or
 * invalidate the capture).  The ordinary entry point `tau_argmax` needs a scratch buffer from the
 * caller; this one keeps its scratch in a fixed array inside the library instead.
 *
 * int tau_argmax_static(const float* logits, int rows, int vocab, int* tokens, int* valid, void* stream)
 *
 *   logits  device pointer, `rows x vocab` 32-bit floats, row-major
 *   tokens  device pointer, `rows` ints: the greatest logit of each row by the total order of
 *           32-bit floats, NaN never chosen, the highest token id among equal logits
 *   valid   device pointer, `rows` ints: 0 for a row that holds only NaN, else 1
 *   stream  a cudaStream_t (0 for the default stream)
 *   returns 0, a CUDA error code (> 0), or a negative code of this header
 *
 * Limits and rules:
 *   - The scratch array holds TAU_ARGMAX_STATIC_WORDS 32-bit words (96 KiB).  Every GPU on which
 *     this library is loaded keeps that much memory until the process ends.  A call needs
 *     `rows * ceil(vocab / 2048) * 3` words; a larger call is refused with
 *     TAU_ARGMAX_STATIC_TOO_LARGE and nothing is launched.  64 rows of a 262,144-token vocabulary fit.
 *   - The first call on each device looks up the array's device address (with that device current)
 *     and remembers it.  Make that first call before any stream capture begins.
 *   - All calls share the one array, and it keeps what the last call wrote.  Its first third holds one
 *     ticket per row, which must be zero when a call's kernel starts: the array is zero when the library
 *     is loaded, every call clears the tickets of its rows in stream order before its kernel (a
 *     cudaMemsetAsync, which allocates nothing), and the kernel puts them back to zero.  The rest may hold
 *     anything: every word of it that the call reads has been written by the same call.  Two calls that
 *     can run at the same time on one GPU (different streams with no ordering between them) race on the
 *     array; order them, or use `tau_argmax` with a scratch buffer per stream.
 *   - No cudaMalloc, cudaFree or other allocating routine is called, on any call.
 */
#pragma once

#define TAU_ARGMAX_STATIC_WORDS 24576
#define TAU_ARGMAX_STATIC_TOO_LARGE (-1)   /* rows * ceil(vocab / 2048) * 3 exceeds TAU_ARGMAX_STATIC_WORDS */
#define TAU_ARGMAX_STATIC_BAD_ARGUMENT (-2) /* a null pointer, or rows or vocab not positive */
#define TAU_ARGMAX_STATIC_BAD_DEVICE (-3)   /* the current device's number is outside the table of remembered addresses */

#ifdef __cplusplus
extern "C" {
#endif
int tau_argmax_static(const float* logits, int rows, int vocab, int* tokens, int* valid, void* stream);
/* Words that a call of this size needs (to compare with TAU_ARGMAX_STATIC_WORDS beforehand). */
long long tau_argmax_static_words_needed(int rows, int vocab);
/* Text for a return value of tau_argmax_static. */
const char* tau_argmax_static_error(int code);
#ifdef __cplusplus
}
#endif
