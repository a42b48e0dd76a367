/*
 * b200q -- C ABI of the B200 (sm_100a) quantized-linear kernels.
 *
 * This is the boundary a host runtime binds instead of the reference's Python /
 * Triton operators.  Each entry point below names the reference routine it
 * stands in for (paths are relative to the reference project).
 *
 * Conventions (modelled on the reference's native runtime ABI,
 * include/linnet/runtime/runtime.h:35-67): every call returns an int32 status
 * (B200Q_OK / B200Q_ERROR / B200Q_UNAVAILABLE); the message of the last failure
 * on the calling thread is read with b200q_last_error().  All pointers are
 * device pointers on the current CUDA device unless stated otherwise; tensors are
 * dense and row-major; sizes are element counts.  `stream` is a cudaStream_t
 * passed as void*.  Unless an entry says otherwise it allocates nothing, never
 * synchronises and keeps no state between calls, so it can be recorded into a
 * CUDA graph and called from several host threads on different streams.  (The
 * library remembers, per kernel and device, that it has raised the kernel's
 * shared-memory limit: one runtime call on first use, none afterwards.)
 */
#ifndef B200Q_H
#define B200Q_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200Q_ABI_VERSION 1

enum { B200Q_OK = 0, B200Q_ERROR = 1, B200Q_UNAVAILABLE = 2 };

/* Element types of activations, scales and outputs. */
enum { B200Q_F32 = 0, B200Q_BF16 = 1, B200Q_F16 = 2 };

int32_t b200q_abi_version(void);

/* Message of the last call that failed on this host thread ("" if none). */
const char* b200q_last_error(void);

/* B200Q_OK when the current device can run these kernels (compute capability
 * 10.x), B200Q_UNAVAILABLE otherwise. */
int32_t b200q_device_ok(void);

/* ---- quantize / pack ------------------------------------------------------
 * Replaces linnet.quant.quantize_int4_groups + pack_int4_groups
 * (python/linnet/src/linnet/quant.py:83-99, :242-248).  Bit-exact.
 *   weight      [out, in], B200Q_F32 or B200Q_BF16 (bf16 is widened exactly)
 *   packed      [out, in/group, group/2] bytes, even k in the low nibble
 *   scale       [out, in/group] f32 (unrounded, as the reference returns it)
 *   scale_store [out, in/group] in `store_dtype`, the value a checkpoint holds
 *               (quant.py:205-209; weights.py:74-79 for bf16); may be NULL
 *   zero        [out, in/group] u8 in 0..15
 * `group` must be even and divide `in`. */
int32_t b200q_quantize_int4_groups(const void* weight, int32_t weight_dtype,
                                   int64_t out, int64_t in, int64_t group,
                                   uint8_t* packed, float* scale,
                                   void* scale_store, int32_t store_dtype,
                                   uint8_t* zero, void* stream);

/* Replaces linnet.quant.quantize_int8_groups (quant.py:102-120).  Bit-exact.
 * The scale is rounded through `scale_dtype` before the levels are chosen;
 * `group == in` gives one scale per output channel.
 *   q     [out, in] i8 in -127..127      scale [out, in/group] f32 */
int32_t b200q_quantize_int8_groups(const void* weight, int32_t weight_dtype,
                                   int64_t out, int64_t in, int64_t group,
                                   int32_t scale_dtype, int8_t* q, float* scale,
                                   void* stream);

/* ---- int4 group-quantized linear ------------------------------------------
 * y[rows, out] = x[rows, in] . dequant(packed, scale, zero)^T, f32 accumulate.
 *   x, y, scale in `dtype` (B200Q_BF16 or B200Q_F16); zero u8.
 * Replaces the torch op linnet::int4_linear
 * (python/linnet/src/linnet/torch/kernels.py:277-323), ATen's
 * _weight_int4pack_mm as the generated source calls it for fewer than 8 rows
 * (src/backend/torch_source.cpp:1556-1558) and the dequantize-then-cuBLAS route
 * for more than 128 rows (:1563-1566).  Picks the kernel from `rows`. */
int32_t b200q_int4_linear(const void* x, const uint8_t* packed, const void* scale,
                          const uint8_t* zero, void* y, int64_t rows, int64_t in,
                          int64_t out, int64_t group, int32_t dtype, void* stream);

/* The decode kernel alone: rows <= 16, HBM-bound weight streaming. */
int32_t b200q_int4_gemv(const void* x, const uint8_t* packed, const void* scale,
                        const uint8_t* zero, void* y, int64_t rows, int64_t in,
                        int64_t out, int64_t group, int32_t dtype, void* stream);

/* Flags of b200q_int4_gemv_ex / b200q_int4_linear_ex (0: the defaults of the entries
 * above).
 *   B200Q_EXACT_WEIGHTS   every weight is (q - zero) * scale computed in f32 and rounded
 *     once to the 16-bit type before the product: bit for bit the weight the reference's
 *     torch path multiplies by (python/linnet/src/linnet/torch/native.py:417-424).
 *     Without the flag, for groups of 128 and one or two rows (where it is the faster
 *     kernel), zero point and scale are applied in f32 to each group's sum of exact
 *     products instead; that is closer to exact arithmetic and differs from the reference
 *     by the rounding noise of its weights (2^-9 relative per weight: sigma 1.4e-3 per
 *     output at K=4096 with weights ~N(0, 0.02) and inputs ~N(0, 1), against the 1e-2
 *     tolerance).  That kernel's weights come through the TMA unit into a ring of
 *     shared-memory stages; its waits on the ring are bounded, and one that expires is
 *     reported by b200q_int4_gemm_status().  The reference selects these kernels under
 *     its `fast` numerics policy only (src/opt/candidates.cpp:28-33).
 *   B200Q_EARLY_DEPENDENTS   the kernels after this one in the stream may start (up to
 *     their own wait on this one's results) as soon as this one has started, instead of
 *     when its last weights are in: pays when the next kernel is another product that can
 *     prefetch its weights meanwhile (q, k, v of one input; a chain of products), costs
 *     when the next kernel only takes room while it waits.
 *   B200Q_SWIGLU_INPUT   x is [rows, 2 in]: the product's input is silu(x[:, :in]) * x[:, in:]
 *     (silu rounded to the 16-bit type, then the product rounded, as the two PyTorch ops of the
 *     reference's generated source do), formed while the kernel stages its activations: the
 *     SwiGLU of a decoder layer without a launch of its own.  Taken for one or two rows,
 *     groups of 128 and the default numerics; B200Q_UNAVAILABLE otherwise (the caller then
 *     forms the input itself).  No counterpart in the reference.
 *   B200Q_NO_OVERLAP   the one- and two-row kernel is launched in plain stream order: it starts
 *     when everything before it in the stream has finished, instead of starting early and
 *     fetching weights while the kernel before it still runs (programmatic dependent launch,
 *     the default).  For callers that want plain stream order, and for timing the kernel
 *     without a neighbour's overlap.  No counterpart in the reference. */
enum { B200Q_EXACT_WEIGHTS = 1, B200Q_EARLY_DEPENDENTS = 2, B200Q_SWIGLU_INPUT = 4, B200Q_NO_OVERLAP = 8 };
int32_t b200q_int4_gemv_ex(const void* x, const uint8_t* packed, const void* scale,
                           const uint8_t* zero, void* y, int64_t rows, int64_t in,
                           int64_t out, int64_t group, int32_t dtype, int32_t flags,
                           void* stream);
int32_t b200q_int4_linear_ex(const void* x, const uint8_t* packed, const void* scale,
                             const uint8_t* zero, void* y, int64_t rows, int64_t in,
                             int64_t out, int64_t group, int32_t dtype, int32_t flags,
                             void* stream);

/* The prefill kernel alone: TMA + tcgen05/TMEM dequant-GEMM (bf16; `in` a multiple of 64,
 * `group` 64 times a power of two, a packed weight under 4 GB; any rows and out;
 * B200Q_ERROR otherwise: b200q_int4_linear sends such shapes to the decode kernels in
 * passes). */
int32_t b200q_int4_gemm(const void* x, const uint8_t* packed, const void* scale,
                        const uint8_t* zero, void* y, int64_t rows, int64_t in,
                        int64_t out, int64_t group, int32_t dtype, void* stream);

/* A decoder layer's residual add, RMS norm and the product that follows, in one launch:
 *   r = x + delta (delta may be null: r = x);   y = (rms_norm(r, eps) * norm_weight) . W^T
 * with W the int4 weight of b200q_int4_gemv and the arithmetic of b200q_add_rmsnorm followed
 * by b200q_int4_gemv (bit for bit, for up to 4096 inputs).  r is stored to x_out (by one block;
 * not when delta is null), which must not be x: every block reads x.  Taken for bf16, one or
 * two rows, groups of 128, up to 8192 inputs and the default numerics; B200Q_UNAVAILABLE
 * otherwise (the caller then runs the two calls).  flags: B200Q_EARLY_DEPENDENTS or 0.  No
 * counterpart in the reference, whose generated source runs the three ops one after another. */
int32_t b200q_int4_gemv_norm(const void* x, const void* delta, const void* norm_weight, float eps,
                             void* x_out, const uint8_t* packed, const void* scale,
                             const uint8_t* zero, void* y, int64_t rows, int64_t in, int64_t out,
                             int64_t group, int32_t dtype, int32_t flags, void* stream);

/* Synchronises the device and reports whether any launch on it of a kernel with a
 * shared-memory pipeline (b200q_int4_gemm, b200q_int8_mm, the one- and two-row kernel of
 * b200q_int4_gemv / b200q_int4_linear) gave up on one of its bounded waits (B200Q_ERROR,
 * with the waiting role in the message); such a launch leaves its output incomplete but the context usable.  Reporting clears
 * the condition (until then later launches cut their waits short).  No reference
 * counterpart: the reference's kernels spin without a bound. */
int32_t b200q_int4_gemm_status(void);

/* Replaces the generated `_int4_weight` / Triton `_int4_unpack`
 * (src/backend/torch_source.cpp:1519-1551): the [out, in] weight in `dtype`,
 * (q - zero) * scale computed in f32 and rounded once. */
int32_t b200q_int4_dequantize(const uint8_t* packed, const void* scale,
                              const uint8_t* zero, void* weight, int64_t out,
                              int64_t in, int64_t group, int32_t dtype, void* stream);

/* ---- int8 weight-only linear ----------------------------------------------
 * y[rows, out] = x[rows, in] . (w * scale)^T, f32 accumulate.
 *   w [out, in] i8; scale f32: [out] when group == 0, else [out, in/group].
 * Replaces linnet::gemv8 (kernels.py:336-434, one row) and linnet::w8a16
 * (kernels.py:437-592, 2..64 rows) for the int8 formats; more rows run the same
 * tiles in passes until the tcgen05 path covers them. */
int32_t b200q_int8_linear(const void* x, const int8_t* w, const float* scale,
                          void* y, int64_t rows, int64_t in, int64_t out,
                          int64_t group, int32_t dtype, void* stream);

/* The same with the flags of b200q_int4_gemv_ex (b200q_int8_linear passes 0).
 *   B200Q_EXACT_WEIGHTS   every weight is w * scale computed in f32 and rounded once to the
 *     16-bit type before the product: the weight the reference's CPU route multiplies by
 *     (python/linnet/src/linnet/torch/quantized.py:193).  Without the flag, for one scale a
 *     row and one or two rows of x, the scale multiplies the finished f32 sum instead, as the
 *     reference's own GPU kernel does (kernels.py:352-371); that kernel's weights come through
 *     the TMA unit, and a bounded wait of it that expires is reported by
 *     b200q_int4_gemm_status().
 *   B200Q_EARLY_DEPENDENTS   as for b200q_int4_gemv_ex. */
int32_t b200q_int8_linear_ex(const void* x, const int8_t* w, const float* scale,
                             void* y, int64_t rows, int64_t in, int64_t out,
                             int64_t group, int32_t dtype, int32_t flags, void* stream);

/* ---- int8 activations x int8 weights (W8A8) ----------------------------------
 * Replaces linnet::rows8 for int8 (python/linnet/src/linnet/torch/kernels.py:669-753):
 * every row of x [rows, in] (`dtype`) gets scale[row] = max(max|row|, 1e-12) / 127 and
 * q[row, :] = x / scale rounded half away from zero, clamped to -127..127; IEEE f32
 * arithmetic.  `in` a multiple of 8. */
int32_t b200q_int8_rows(const void* x, int8_t* q, float* scale, int64_t rows, int64_t in,
                        int32_t dtype, void* stream);

/* Replaces linnet::int8_mm (kernels.py:805-915): y[rows, out] in `dtype` =
 * (xq . w^T summed exactly in int32) * x_scale[row] * w_scale[col], tcgen05 kind::i8 with the
 * accumulator in tensor memory.  xq [rows, in] and w [out, in] int8, `in` a multiple of
 * 128, both 16-byte aligned.  A bounded wait that expires is reported by
 * b200q_int4_gemm_status(). */
int32_t b200q_int8_mm(const int8_t* xq, const int8_t* w, const float* x_scale,
                      const float* w_scale, void* y, int64_t rows, int64_t in, int64_t out,
                      int32_t dtype, void* stream);

/* Replaces dequantize8 (kernels.py:595-666) for int8: weight[out, in] in `dtype`
 * = round(f32(w) * scale). */
int32_t b200q_int8_dequantize(const int8_t* w, const float* scale, void* weight,
                              int64_t out, int64_t in, int64_t group, int32_t dtype,
                              void* stream);

/* ---- decode-step glue ------------------------------------------------------
 * The small operations between the quantized linears of a decode step.  In the
 * reference they are stdlib ops lowered to PyTorch calls inside the captured
 * decode graph (examples/01-llama/src/lib.linnet and attention.linnet, replayed by
 * python/linnet/src/linnet/torch/compiled.py:430-503): rms_norm, rope, the
 * index_put_ cache write, scaled_dot_product_attention, silu * mul.  All tensors
 * are bf16 unless stated. */

/* x[rows, hidden] += delta (skipped when delta is NULL), then
 * y = x * rsqrt(mean(x^2) + eps) * weight, computed in f32. */
int32_t b200q_add_rmsnorm(void* x, const void* delta, const void* weight, void* y,
                          int64_t rows, int64_t hidden, float eps, void* stream);

/* qkv [batch, (nq + 2 nkv) * head_dim]: rotary embedding (halves rotated) of the
 * query and key heads at positions[batch] (int64); queries go to q_out
 * [batch, nq, head_dim], keys and values to cache_{k,v}[batch, nkv, max_seq,
 * head_dim] at their position.
 * Positions are device data, so they are checked on the device, here and in the
 * attention entries below: a position outside 0 .. max_seq-1 stores nothing for that
 * row, forms no address outside the caches, and is recorded for
 * b200q_decoder_status().  The caches must hold finite values everywhere (fill them
 * with zeros once): a tile of keys and values is read whole. */
int32_t b200q_rope_cache(const void* qkv, const int64_t* positions, void* q_out,
                         void* cache_k, void* cache_v, int64_t batch, int64_t nq,
                         int64_t nkv, int64_t head_dim, int64_t max_seq, float theta,
                         void* stream);

/* Single-query attention of q [batch, nq, head_dim] over cache positions
 * 0..positions[b], grouped-query (nq / nkv in 1, 2, 4, 8; head_dim 64 or 128), the
 * keys split `splits` ways.  `scratch` is caller-owned device memory of
 * b200q_decode_attention_scratch_bytes(...) bytes holding the splits' partial
 * results; out is [batch, nq * head_dim]. */
int64_t b200q_decode_attention_scratch_bytes(int64_t batch, int64_t nq, int64_t head_dim,
                                             int64_t splits);
int32_t b200q_decode_attention(const void* q, const void* cache_k, const void* cache_v,
                               const int64_t* positions, void* out, void* scratch,
                               int64_t batch, int64_t nq, int64_t nkv, int64_t head_dim,
                               int64_t max_seq, int64_t splits, void* stream);


/* Rotary embedding + cache write + attention in one launch (b200q_rope_cache followed by
 * b200q_decode_attention_cluster): `qkv` is the fused projection [batch, (nq + 2 nkv) *
 * head_dim] of this step; `rope` is a table [max_seq, head_dim / 2] of (cos, sin) f32 pairs
 * filled once by b200q_rope_table (the same arithmetic as b200q_rope_cache).  The queries are
 * rotated in registers; the block whose keys end at positions[b] rotates the new key, puts it
 * and the new value into its tile and writes both to the caches.  1 to 8 splits.  No
 * reference counterpart (the reference runs PyTorch ops here). */
int32_t b200q_rope_table(void* table, int64_t max_seq, int64_t head_dim, float theta, void* stream);
int32_t b200q_rope_attention(const void* qkv, const int64_t* positions, const void* rope,
                             void* cache_k, void* cache_v, void* out, int64_t batch, int64_t nq,
                             int64_t nkv, int64_t head_dim, int64_t max_seq, int64_t splits,
                             void* stream);

/* b200q_decode_attention in one launch and without scratch: the `splits` (1 to 8) blocks
 * of a (row, kv head) form one thread-block cluster and merge their partial results through
 * distributed shared memory.  Allocates nothing.  No reference counterpart: the reference
 * runs PyTorch's attention here. */
int32_t b200q_decode_attention_cluster(const void* q, const void* cache_k, const void* cache_v,
                                       const int64_t* positions, void* out, int64_t batch,
                                       int64_t nq, int64_t nkv, int64_t head_dim,
                                       int64_t max_seq, int64_t splits, void* stream);
/* b200q_decode_attention for hosts that cannot give it scratch memory (a runtime with a
 * fixed arena, a plug-in without access to the allocator, a caller inside a stream
 * capture): the partial results go to a 4 MiB array built into the library, which every
 * GPU that loads the library holds until the process exits.  It has no counterpart in
 * the reference.  Same arguments and result as b200q_decode_attention without `scratch`.
 *   - Fails with B200Q_ERROR when b200q_decode_attention_scratch_bytes(batch, nq,
 *     head_dim, splits) exceeds b200q_decode_attention_static_scratch_limit().
 *   - The first call on each device looks the array's address up (one runtime query, no
 *     allocation); make that first call before you begin capturing a stream.
 *   - All calls share the one array and it keeps the previous call's contents (nothing in
 *     it needs clearing: every partial result read was written by the same call), so two
 *     calls whose kernels overlap on the GPU -- different streams, or graphs replayed
 *     side by side -- race; keep them ordered.
 *   - Allocates nothing, frees nothing. */
int64_t b200q_decode_attention_static_scratch_limit(void);
int32_t b200q_decode_attention_static(const void* q, const void* cache_k, const void* cache_v,
                                      const int64_t* positions, void* out, int64_t batch,
                                      int64_t nq, int64_t nkv, int64_t head_dim, int64_t max_seq,
                                      int64_t splits, void* stream);

/* Synchronises the device and reports (B200Q_ERROR, naming the batch row) whether a
 * decode-step kernel since the last report met a position outside its cache; reporting
 * clears the condition.  No reference counterpart (PyTorch's index_put_ raises a
 * device-side assertion there). */
int32_t b200q_decoder_status(void);

/* out[rows, inner] = silu(gate_up[:, :inner]) * gate_up[:, inner:], silu rounded to
 * bf16 before the product as the two PyTorch ops round. */
int32_t b200q_silu_mul(const void* gate_up, void* out, int64_t rows, int64_t inner,
                       void* stream);

/* Tensor-parallel epilogue of a row-split layer in one launch: all-reduce of the ranks'
 * partial sums over NVLink peer memory, residual add and RMSNorm:
 *     x[rows, hidden] += bf16(sum over ranks of partial_r[rows, hidden]);  y = rms_norm(x) * weight
 * Replaces `std.nn.parallel::all_reduce` after a `Shards` layer (stdlib/nn/parallel.linnet:9-11;
 * the reference's one-shot route: python/linnet/src/linnet/torch/collectives.py:145-167,
 * kernel python/linnet/src/linnet/torch/kernels.py:1107-1156) plus the residual add and norm
 * that follow it in a decoder layer.  bf16 only.
 *   peer_areas: HOST array of `world` device addresses, all mapped into this process
 *     (symmetric / peer memory): rank r's receive area of this call site, [world][slot_words]
 *     words of 8 bytes (two bf16 values + the call's 32-bit epoch; each word is stored and
 *     polled as one 64-bit element, which is what makes values and epoch arrive together),
 *     slot_words >= rows * hidden / 2 and even, 16-byte aligned, zeroed once.
 *   partial: this rank's partial sums [rows, hidden] (local memory, 16-byte aligned), written
 *     by this rank's own kernels earlier in the stream.  The kernel stores them, each word
 *     tagged with the epoch, into slot `rank` of every peer's area and reads the peers' words
 *     from its own area, polling each until its epoch matches.
 *   epoch, done: this rank's uint32 counters of this call site (zeroed once); error: an int32
 *     the kernel sets to 100+r when rank r's words did not arrive within the wait limit (the
 *     kernel then returns without reducing; the context stays usable, and later calls do not
 *     wait at all until the host has zeroed the word).
 * Every rank must make the same sequence of calls per site; a site may be used again only
 * after a call on a DIFFERENT site has been issued in between (a decoder has 2 per layer).
 * Plain peer stores and local loads only; no barrier, fence or flag between the ranks. */
int32_t b200q_tp_allreduce_add_rmsnorm(const int64_t* peer_areas, int64_t slot_words,
                                       const void* partial, int32_t world, int32_t rank,
                                       void* epoch, void* done, void* error, void* x,
                                       const void* weight, void* y, int64_t rows, int64_t hidden,
                                       float eps, void* stream);

/* The exchange of b200q_tp_allreduce_add_rmsnorm alone: out[count] = the ranks' in[count]
 * summed in f32 in rank order and rounded once to `dtype` (bf16 or f16), count a multiple
 * of 8.  Replaces the reference's one-shot all-reduce for messages up to 128 KiB
 * (`OneShot.__call__`, python/linnet/src/linnet/torch/collectives.py:86-103; kernel
 * kernels.py:1107-1156), with every wait bounded.  Same areas, counters, error word and
 * call-site rule as above (slot_words >= count / 2). */
int32_t b200q_tp_allreduce(const int64_t* peer_areas, int64_t slot_words, const void* in,
                           int32_t world, int32_t rank, void* epoch, void* done, void* error,
                           void* out, int64_t count, int32_t dtype, void* stream);

/* b200q_tp_allreduce_add_rmsnorm with a different exchange: rows pushed as plain bf16, then
 * one flag per (source rank, row).  peer_areas[r]: rank r's receive area of the call site,
 * [world][slot_elems] bf16 with slot_elems >= max_rows * hidden; peer_flags[r]: rank r's flag
 * words of the site, [world][max_rows] uint32, zeroed once.  This rank's partial sums are
 * written (by its own kernels, earlier in the stream) into slot `rank` of its OWN area.
 * Same arithmetic, counters, error code and call-site rule.  Faster than the tagged words from
 * about four ranks up (half the NVLink bytes), slower on two.  No reference counterpart beyond
 * the all_reduce both replace. */
int32_t b200q_tp_allreduce_add_rmsnorm_flags(const int64_t* peer_areas, const int64_t* peer_flags,
                                             int64_t slot_elems, int64_t max_rows, int32_t world,
                                             int32_t rank, void* epoch, void* done, void* error,
                                             void* x, const void* weight, void* y, int64_t rows,
                                             int64_t hidden, float eps, void* stream);

/* How long the two tensor-parallel kernels above wait for a peer before they give up:
 * process-wide, read at launch; one second unless set.  No reference counterpart (the
 * reference's one-shot all-reduce spins without a bound, kernels.py:1146-1148). */
int32_t b200q_set_wait_limit_ns(int64_t nanoseconds);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H */
