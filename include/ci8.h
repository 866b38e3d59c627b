/*
 * C ABI of the sm_100a W8A8 linear kernels (libci8.so).
 *
 * Every entry point takes raw DEVICE pointers, plain sizes and a CUDA stream, launches on that
 * stream and returns immediately: no allocation, no host synchronisation, no device-to-host
 * read, so each call can be captured in a CUDA graph. Outputs are caller-owned and written in
 * place. Return value: 0 on success, otherwise a cudaError_t value (cudaErrorInvalidValue = 1
 * for rejected arguments); nothing is thrown across this boundary. ci8_error_string() turns a
 * code into text. The torch stable-ABI operators in csrc/bindings.cpp are thin wrappers over
 * these functions; they replace the reference's host launchers declared in csrc/kernels.h.
 *
 * Matrices are row-major and contiguous. "BF16" is the 16-bit bfloat16 bit pattern.
 */
#ifndef CI8_H_
#define CI8_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* ci8_stream_t;

/* Replaces quantize_rows (reference csrc/kernels.h:48-49, csrc/kernels.cu:283-292).
 * x BF16 [m,k] -> codes INT8 [m,k], scales FP32 [m].
 * scale = max(absmax/127, 1e-20); code = clamp(round_half_even(x/scale), -127, 127). m,k > 0. */
int ci8_quantize_rows(const void* x, int8_t* codes, float* scales, int m, int k,
                      ci8_stream_t stream);

/* Replaces quantize_grouped4096 (reference csrc/kernels.h:50-51, csrc/kernels.cu:293-298; C-ABI
 * precedent benchmarks/cuda/grouped_quant4096.cu:56-62).
 * x BF16 [m,groups,4096] -> codes INT8 [groups,m,4096], scales FP32 [groups,m]. m == 0 is a
 * no-op. x must be 16-byte aligned, codes 8-byte aligned. */
int ci8_quantize_grouped4096(const void* x, int8_t* codes, float* scales, int m, int groups,
                             ci8_stream_t stream);

/* Replaces unpack_allspark (reference csrc/kernels.h, csrc/allspark_layout.cu:8-35): packed UINT8
 * [ceil(n/32)*32, k] in AllSpark N32K16 order with permuted BF16 packed_scales [ceil(n/32)*32] ->
 * weight INT8 [n,k] (code - 128, row-major) and scales BF16 [n]. n % 16 == 0, k % 16 == 0,
 * k <= 65536; packed and weight 16-byte aligned (the reference asks 4 bytes of packed). */
int ci8_unpack_allspark(const uint8_t* packed, const void* packed_scales, int8_t* weight,
                        void* scales, int n, int k, ci8_stream_t stream);

/* Replaces silu_mul (reference csrc/silu_quant.h, csrc/silu_quant.cu:64-88): x BF16 [m, 2k] holds
 * gate | up per row; out BF16 [m,k] = bf16(silu(gate) * up), silu = gate / (1 + expf(-gate)).
 * The reference accepts k = 8704 or 17408; any k % 8 == 0 is accepted here. 16-byte aligned. */
int ci8_silu_mul(const void* x, void* out, int m, int k, ci8_stream_t stream);

/* Replaces silu_mul_quantize (reference csrc/silu_quant.cu:10-62,77-83): the same SwiGLU fused in
 * front of the row quantizer; bit-identical to ci8_silu_mul followed by ci8_quantize_rows.
 * codes INT8 [m,k], scales FP32 [m]; k % 8 == 0, k <= 65536; x 16-byte, codes 8-byte aligned. */
int ci8_silu_mul_quantize(const void* x, int8_t* codes, float* scales, int m, int k,
                          ci8_stream_t stream);

/* Replaces fused_channel_mm (reference csrc/kernels.h:27-29, csrc/fused_mm.cu:66-93).
 * a INT8 [m,k], w INT8 [n,k], a_scale FP32 [m], w_scale BF16 [n] -> out BF16 [m,n],
 * out = bf16((float(sum_k a*w) * a_scale[row]) * float(w_scale[col])).
 * k % 32 == 0, k <= 65536, a and w 16-byte aligned. schedule in [0,6]: 0 = automatic; other
 * values select a tile configuration; every schedule produces identical bits. */
int ci8_fused_channel_mm(const int8_t* a, const int8_t* w, const float* a_scale,
                         const void* w_scale, void* out, int m, int n, int k, int schedule,
                         ci8_stream_t stream);

/* Replaces cutlass_channel_mm (reference csrc/kernels.h:63-65, csrc/cutlass_mm.cu:39-50).
 * As ci8_fused_channel_mm, and the exact INT32 accumulators are also written to
 * workspace INT32 [m,n] (caller-owned). */
int ci8_cutlass_channel_mm(const int8_t* a, const int8_t* w, const float* a_scale,
                           const void* w_scale, int32_t* workspace, void* out, int m, int n,
                           int k, ci8_stream_t stream);

/* Replaces channel_mm (reference csrc/kernels.h:56-58, csrc/kernels.cu:299-303).
 * w UINT8 [n,k] holds signed code + 128. Any n > 0; k % 32 == 0, k <= 65536. a and w need 4-byte
 * alignment only, as in the reference (it reads 32-bit words, csrc/kernels.cu:99,105); operands that
 * are not 16-byte aligned run a plain word-wise kernel with the same bits, much slower than the
 * tensor-core paths the aligned ones take. */
int ci8_channel_mm(const int8_t* a, const uint8_t* w, const float* a_scale, const void* w_scale,
                   void* out, int m, int n, int k, ci8_stream_t stream);

/* Replaces channel_gemv (reference csrc/kernels.h:54-55, csrc/gemv.cu:50-59). W8A16:
 * x BF16 [m,k], w INT8 [n,k], w_scale BF16 [n] -> out BF16 [m,n] with
 * out = bf16(sum_k x * bf16(float(w) * float(w_scale))), FP32 accumulation.
 * 0 < m <= 16 (the reference stops at 8), k % 16 == 0, k <= 65536, w 16-byte aligned. */
int ci8_channel_gemv(const void* x, const int8_t* w, const void* w_scale, void* out, int m,
                     int n, int k, ci8_stream_t stream);

/* Grouped-scale W8A8 in one launch. The reference composes this from quantize_grouped4096 and
 * one fused_channel_mm per group (benchmarks/benchmark_grouped_w8a8.py:100-107); its precedent
 * for FP32-summed rescaled INT32 partials is benchmarks/cuda/q8_block_int8.cu:44-62.
 * codes INT8 [groups,m,4096] and scales FP32 [groups,m] as written by
 * ci8_quantize_grouped4096; w INT8 [n, groups*4096]; w_scale BF16 [n] -> out BF16 [m,n]:
 * out = bf16((sum over g ascending of float(acc_g) * scales[g,row]) * float(w_scale[col])),
 * FP32 multiply and add rounded separately. With groups == 1 this is ci8_fused_channel_mm. */
int ci8_grouped_channel_mm(const int8_t* codes, const int8_t* w, const float* scales,
                           const void* w_scale, void* out, int m, int n, int groups,
                           ci8_stream_t stream);

/* ci8_grouped_channel_mm with a caller-lent workspace (no counterpart in the reference). When the tiles
 * of the last wave would leave most of the GPU idle (M = 2048, N = 7168 on 148 SMs: 224 tiles of 256 x 256
 * for 74 CTA pairs, so two tiles in a fourth wave), those tiles are cut along the groups: every group of
 * such a tile runs on a CTA pair of its own (the pairs that finish their whole tiles first draw the
 * pieces from a counter in the workspace), writes its FP32 terms to the workspace, and the pairs then
 * add the terms in ascending group order, the same fadd chain as without the split, so the output
 * has the same bits. ci8_grouped_workspace_bytes() tells how much the shape needs on the current device
 * (0: the split would not pay and no workspace is used). The workspace must be 16-byte aligned and
 * ZERO before its first use; the kernel leaves its counters zero again, so it can be reused by later
 * calls in the same stream (not by calls that may overlap). A NULL or too small workspace gives the
 * plain ci8_grouped_channel_mm. */
long long ci8_grouped_workspace_bytes(int m, int n, int groups);
int ci8_grouped_channel_mm_ws(const int8_t* codes, const int8_t* w, const float* scales,
                              const void* w_scale, void* out, void* workspace,
                              long long workspace_bytes, int m, int n, int groups,
                              ci8_stream_t stream);

/* quantize_rows followed by fused_channel_mm as one call (reference csrc/kernels.cu:283-292 then
 * csrc/fused_mm.cu:66-93; the reference always launches the two separately). x BF16 [m,k], w INT8
 * [n,k], w_scale BF16 [n] -> out BF16 [m,n]; codes INT8 [m,k] and scales FP32 [m] receive exactly what
 * ci8_quantize_rows would write (caller-owned, also usable afterwards). For m <= 16 and k <= 8192, when
 * the streaming kernel runs unsplit, this is ONE kernel: every CTA derives the row scales from the
 * activations and quantizes each K block on its way into the MMA operand tile, so the quantizer's
 * launch disappears from the decode step; otherwise the two kernels are launched back to back. The
 * results are bit-identical either way. x, codes and w 16-byte aligned; k % 32 == 0. */
int ci8_dynamic_channel_mm(const void* x, const int8_t* w, const void* w_scale, int8_t* codes,
                           float* scales, void* out, int m, int n, int k, ci8_stream_t stream);

/* The gate/up projection with the SwiGLU fused into its epilogue. No single counterpart in the
 * reference: it replaces fused_channel_mm (csrc/fused_mm.cu:66-93) followed by silu_mul
 * (csrc/silu_quant.cu:64-88) and produces the same bits as that pair, without writing and re-reading
 * the [m, n] BF16 intermediate. w INT8 [n, k] and w_scale BF16 [n] hold gate and up rows interleaved
 * in blocks of 128: rows [256t, 256t+128) are gate channels [128t, 128t+128), rows [256t+128, 256t+256)
 * the up channels of the same range (consumer_int8.quantization.interleave_gate_up builds this order
 * from the [gate | up] layout). out BF16 [m, n/2] = bf16(silu(gate) * up) with gate and up rounded to
 * BF16 first, as the unfused pair does. n % 256 == 0, k % 32 == 0; a, w and out 16-byte aligned. */
int ci8_gate_up_silu_mm(const int8_t* a, const int8_t* w, const float* a_scale, const void* w_scale,
                        void* out, int m, int n, int k, ci8_stream_t stream);

/* Replaces q8_block_int8 (reference benchmarks/cuda/q8_block_int8.cu:150-160, a raw C entry point
 * bound with ctypes by benchmarks/benchmark_q8_block_int8.py:36-39; same argument order). Block-32
 * (GGUF Q8_0) W8A8: x BF16 [m,k] is quantized per 32 values into a INT8 [m,k] with sa FP32
 * [m,k/32] (both caller-owned scratch that is also an output), then
 * y[m,n] = bf16(sum over blocks b ascending of fma(float(dot_b), sa[m,b] * float(sw[n,b]), .)),
 * dot_b the INT32 product of the block's 32 codes; w INT8 [n,k] (codes in [-128,127]), sw FP16
 * [n,k/32], y BF16 [m,n]. k % 32 == 0, k <= 65536; x, a and w 16-byte aligned. */
int ci8_q8_block_mm(const void* x, int8_t* a, float* sa, const int8_t* w, const void* sw, void* y,
                    int m, int n, int k, ci8_stream_t stream);

/* ci8_q8_block_mm under the reference's own symbol name (benchmarks/cuda/q8_block_int8.cu:150-160):
 * the reference's validation script (benchmarks/benchmark_q8_block_int8.py:36-39,253-257) accepts no
 * other entry name, so with this alias `--library libci8.so` is the only change to its command line. */
int q8_block_int8(const void* x, int8_t* a, float* sa, const int8_t* w, const void* sw, void* y,
                  int m, int n, int k, ci8_stream_t stream);

/* ci8_q8_block_mm for callers that have no device memory to hand over. It has no counterpart in the
 * reference. ci8_q8_block_mm needs two caller-owned scratch buffers (the activation codes and their
 * block scales); some callers cannot provide them: a plugin that runs inside a serving engine whose
 * memory pool already owns the whole GPU (a cudaMalloc there fails or fragments the pool), code that
 * runs while a stream is being captured (allocation is not allowed then), or a host that simply has no
 * allocator wired up. This variant keeps that scratch inside the library instead: a fixed array in
 * device memory (4.5 MiB, present on every GPU that loads the library until the process exits). It
 * calls no cudaMalloc / cudaFree and no allocating library routine. Inputs x, w, sw and the output y
 * are as for ci8_q8_block_mm and still belong to the caller.
 *   Limit: m * k <= ci8_q8_block_static_max_values() (4 Mi values, e.g. 1024 rows of K = 4096);
 *   anything larger is rejected with cudaErrorInvalidValue before any launch.
 *   First use: the first call on each device looks up the array's device address (with that device
 *   current); make that call once before capturing a stream.
 *   Sharing: every call on a device uses the same array. Calls are safe back to back on one stream;
 *   calls that may run at the same time on the GPU (two streams, two host threads) overwrite each
 *   other's codes and give wrong results. Nothing has to be cleared between calls: each call writes
 *   every code and scale it later reads. The array's contents after a call are unspecified. */
int ci8_q8_block_mm_static(const void* x, const int8_t* w, const void* sw, void* y, int m, int n, int k,
                           ci8_stream_t stream);
int ci8_q8_block_static_max_values(void);

/* fused_channel_mm for an output-channel shard, with the all-gather of the result fused into the
 * GEMM's epilogue. The reference has no collective (its serving stack gathers column-parallel
 * results outside the library, benchmarks/microbench.py:187); this entry point replaces
 * "fused_channel_mm then all-gather". gathered[r] (r = 0..world-1, a HOST array of device
 * pointers) is rank r's BF16 buffer [world, m, n_shard], peer-mapped into this process; this
 * rank's [m, n_shard] result is written into block `rank` of every one of them with TMA tile
 * stores issued as each tile finishes, so the NVLink transfers overlap the main loop. The caller
 * must order a cross-rank barrier after this call before any rank reads its buffer.
 * w INT8 [n_shard, k] is this rank's slice of the weight; n_shard % 8 == 0; world <= 8. Of `schedule`
 * only the choice between one-CTA (odd) and two-CTA (even) tiles is honoured: the tile width is
 * chosen among those that are whole 64-column store boxes. */
int ci8_fused_channel_mm_gather(const int8_t* a, const int8_t* w, const float* a_scale,
                                const void* w_scale, void* const* gathered, int world, int rank,
                                int m, int n_shard, int k, int schedule, ci8_stream_t stream);

/* ci8_fused_channel_mm_gather with the closing cross-GPU barrier inside the kernel (no counterpart in
 * the reference). signals[r] (a HOST array of device pointers, r = 0..world-1) points to 8 arrival
 * counters of 8 bytes each in rank r's memory, peer-mapped into this process like the gathered
 * buffers, zero before the first call and never reset; state points to 32 zero-initialised bytes in
 * THIS rank's memory (calls completed, CTAs gone, tiles drawn: after its first tile a worker of this
 * form draws its next tile from a counter, because the CTAs do not get equal shares of a saturated
 * link; one spare word). Every CTA signals every rank after its stores have landed and then waits until
 * all CTAs of all ranks have signalled this rank, so when the kernel ends the whole gathered result
 * is in this rank's buffer: no collective has to follow. All ranks must make the same sequence of
 * calls on one set of (gathered, signals, state). A rank may start call i+1 on a set while a peer
 * still reads the result of call i from it, so alternate two sets when results are read between
 * calls (call i+2 on a set cannot start before every rank has finished call i+1 on the other set,
 * which orders it after every read of call i). A peer that never arrives ends the wait after 2 s
 * with status bit 2 set (ci8_device_status); the call count still advances. Capturable in a CUDA
 * graph: the call counter lives in `state`, not in the arguments. */
int ci8_fused_channel_mm_gather_sync(const int8_t* a, const int8_t* w, const float* a_scale,
                                     const void* w_scale, void* const* gathered, void* const* signals,
                                     void* state, int world, int rank, int m, int n_shard, int k,
                                     int schedule, ci8_stream_t stream);

/* The closing barrier of ci8_fused_channel_mm_gather as a one-thread kernel of its own (no counterpart
 * in the reference): ordered after the gathering GEMM in the stream, it tells every peer that this
 * rank's stores are complete and waits until every peer has said the same, so that what follows in
 * the stream sees the whole gathered result. signals and state as for
 * ci8_fused_channel_mm_gather_sync (each caller needs its own state and counters: do not share them
 * with that entry point). Bounded like every wait: 2 s, then status bit 2. */
int ci8_peer_rendezvous(void* const* signals, void* state, int world, int rank, ci8_stream_t stream);

/* The streaming (m <= 64) kernel behind ci8_fused_channel_mm / ci8_cutlass_channel_mm /
 * ci8_channel_mm with the split-K factor forced to 1, 2 or 4 (1 or 2 for m > 16) instead of chosen
 * from the shape.
 * No counterpart in the reference; it exists so that tests can show the result does not depend
 * on the split. weights_biased != 0: w is UINT8 code+128. workspace may be NULL. */
int ci8_decode_mm_split(const int8_t* a, const void* w, const float* a_scale, const void* w_scale,
                        int32_t* workspace, void* out, int m, int n, int k, int split,
                        int weights_biased, ci8_stream_t stream);

/* Diagnostic, no launch and no counterpart in the reference: the tiling ci8_fused_channel_mm (groups
 * == 1, schedule 0) or ci8_grouped_channel_mm (groups > 1, k = 4096) would use for this shape on the
 * current device. plan[0] = channels per tile, plan[1] = channel tiles per row stripe, plan[2] = how
 * many of those are 32 channels wider than plan[0] (the mixed-width form), plan[3] = column slices
 * the tiles of the last wave are cut into. Tests use it to make sure every form is exercised. */
int ci8_gemm_tile_plan(int m, int n, int k, int groups, int* plan);

/* Diagnostic (no counterpart in the reference): output channels per tile (64, 32 or 16) the block-32
 * kernel takes for an [m, n] result on the current device, or 0 for a bad argument. Tests use it to make
 * sure every width is exercised. */
int ci8_q8_block_tile_channels(int m, int n);

/* Self-test of the kernels' bounded waits (no counterpart in the reference): launches one CTA that
 * waits on a barrier nothing arrives on; after deadline_us microseconds (1..1000000) the wait
 * gives up exactly as the production kernels' waits do after their 2 s deadline: status bit 0 is
 * raised, *gave_up (a device int) is set to 1 and the kernel returns, leaving the context usable. */
int ci8_selftest_wait_timeout(unsigned deadline_us, int* gave_up, ci8_stream_t stream);

/* The same for the rendezvous between the CTAs of a cluster (the split-K streaming kernel's leader
 * waits for its peers' partial sums on a barrier they arrive on remotely): launches one 2-CTA cluster
 * whose second CTA never arrives; after deadline_us the first CTA gives up, status bit 1 is raised,
 * *gave_up is set to 1 and both CTAs leave through their closing cluster barrier. Nothing traps. */
int ci8_selftest_cluster_timeout(unsigned deadline_us, int* gave_up, ci8_stream_t stream);

/* Reads and clears the current device's kernel status word (synchronises the device). Bit 0: a
 * bounded wait inside a kernel ran past its deadline and the kernel gave up (its output is then
 * undefined); bit 1: a cluster rendezvous did; bit 2: the cross-GPU rendezvous of
 * ci8_fused_channel_mm_gather_sync did (a peer never arrived). Returns 0 or a cudaError_t. Not for use during stream capture. */
int ci8_device_status(unsigned* status);

/* The same check without a synchronisation, for serving loops that replay CUDA graphs (no counterpart in
 * the reference): enqueues a one-thread kernel that ORs the status word into *word and clears it. word
 * is caller-owned, 4-byte aligned, device memory or pinned host memory mapped into the device; it is
 * only ever ORed into, so the host may read it at any time and clear it when it has acted on it. Put
 * one such call at the end of a captured step and poll the word every few steps: a non-zero value means
 * that a kernel of an earlier step gave up on a wait and that step's output is not to be trusted. */
int ci8_device_status_async(unsigned* word, ci8_stream_t stream);

/* Text for a code returned by any function above. */
const char* ci8_error_string(int code);

/* Library ABI version (bumped when a signature changes). */
int ci8_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* CI8_H_ */
