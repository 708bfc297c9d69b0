/* Entry points of _pear_kernels.so that allocate nothing, for callers that cannot allocate device memory at call time.
 *
 * Who needs this: code that runs inside a region where the CUDA allocator must not be touched -- a latency-critical
 * serving loop that has handed all free memory to a KV cache, a host thread that is not allowed to take the allocator's
 * lock, an embedder written in C that has no tensor library at all. The regular entry point `pear_fused_sample` takes its
 * workspace from the caller (the Python binding gets it from torch's allocator on every call); the variant below keeps
 * the workspace in a fixed array inside the library's own device image instead.
 *
 * (This entry point has no counterpart in the upstream project.)
 */
#ifndef PEAR_NO_ALLOC_H
#define PEAR_NO_ALLOC_H

#ifdef __cplusplus
extern "C" {
#endif

/* Limits of the built-in workspace: rows * chunks chunk records of 288 bytes (288 KiB in total). */
#define PEAR_SAMPLE_STATIC_MAX_ROWS 64
#define PEAR_SAMPLE_STATIC_MAX_RECORDS 1024

/* Error codes besides cudaError_t values (which are positive). */
#define PEAR_NOALLOC_TOO_LARGE (-2) /* rows > MAX_ROWS or rows * chunks > MAX_RECORDS: use pear_fused_sample instead */
#define PEAR_NOALLOC_BAD_ARGUMENT (-3) /* topk outside 1..32, chunks outside 1..64, temperature <= 0 */

/* Temperature-only sampling of `rows` rows of fp32 logits [rows, ld] (exponential race with the caller's uniform noise
 * [rows, V]), with the sampled token's log-prob, the top-`topk` log-probs and ids, the token's rank and the count of
 * NaN / +inf logits per row: the same results as pear_fused_sample, bit for bit.
 *
 * - Allocates nothing: no cudaMalloc / cudaFree, no library call that allocates. All outputs are caller-provided device
 *   buffers (tok, rank, nonfinite: int[rows]; tok_lp: float[rows]; top_id: int[rows * topk]; top_lp: float[rows * topk]).
 * - Set-up: the FIRST call on each device looks up the address of the built-in workspace (cudaGetSymbolAddress). Make
 *   that first call before any stream capture begins on that device.
 * - Nothing has to start at zero: every workspace record a call reads was written earlier in the same call.
 * - The workspace is one per device and shared by all callers: two calls that overlap in time on one device (different
 *   streams or threads) race on it. Serialise them, or use pear_fused_sample with separate workspaces.
 * - Sizes beyond the limits above are refused with PEAR_NOALLOC_TOO_LARGE before anything is launched.
 *
 * Returns 0, a cudaError_t (> 0), or one of the negative codes above. */
int pear_fused_sample_static(const float* logits, int rows, int V, int ld, float temperature, const float* noise, int chunks,
                             int topk, int* tok, float* tok_lp, int* top_id, float* top_lp, int* rank, int* nonfinite,
                             void* stream);

#ifdef __cplusplus
}
#endif
#endif
