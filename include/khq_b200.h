/*
 * khq_b200.h -- C ABI of libbonsai_khq_b200.so: Bonsai-27B full-attention path over a
 * KHQ-compressed KV cache, hand-written for NVIDIA B200 (sm_100a).
 *
 * Section 1 re-exports, with identical names, argument order and meaning, the entry points the
 * reference host binds by dlsym() for this path (reference paths are relative to the reference
 * project's root).  Section 2 are additions the reference has no counterpart for (batching,
 * fusion, context-parallel partials, prefill).
 *
 * Conventions shared by every launcher, as in the reference:
 *   - returns int: 0 = enqueued; negative = contract violation (nothing was launched);
 *     positive = the cudaError_t reported by cudaGetLastError() after the launch;
 *   - the last argument is the CUDA stream to launch on (the reference host passes NULL);
 *   - every pointer is a DEVICE pointer owned by the caller; launchers allocate nothing, never
 *     synchronise and keep no reference to the buffers after the kernels have run;
 *   - shapes are Bonsai-27B's attention: head_dim D = 256, H_q = 24, H_kv = 4 (n_rep = 6),
 *     rotary dims 0..63 in half-split pairs (m, m+32).  Other H_kv / n_rep return -103.
 *
 * Fixed byte layouts (rows are token-major with the kv-heads interleaved: row = token*H_kv + kv):
 *   k_mask        (rows, 16) uint32   2-bit symbol per dim, dim i at bits 2*(i%16) of word i/16
 *   k_payload     (rows, 40) uint8    [0:4] u32 base multiplier*1000, [4:29] 4-bit outlier
 *                                     residuals, [29:36] outlier sign bits, [36] 0x02, [37:40] 0
 *   v_payload     (rows, 104) uint8   24 words of 8x12-bit patch fields + 2 words of VQ bit 7
 *   *_norms, *_r_norms (rows) fp16;   v_shared_meta (rows) fp32 stored in 4 bytes
 *   q / q_gate    (H_q, 2*D) fp16     query at [0,D), output-gate logits at [D,2D) of each head
 *   partial/attn  (.., D+2) fp32      unnormalised accumulator[D], running max, sum of exps
 */
#ifndef KHQ_B200_H_
#define KHQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef KHQ_B200_STREAM_T
#define KHQ_B200_STREAM_T
typedef struct CUstream_st* khq_stream_t; /* == cudaStream_t */
#endif

/* ------------------------------------------------------------------------------------------
 * Section 1: drop-in replacements for the reference's FFI symbols
 * ---------------------------------------------------------------------------------------- */

/* Replaces bonsai_cuda_sm75_init (src/csrc/qmv_sm75_kernel.cu:3974). Always 0. */
int bonsai_cuda_sm75_init(void);

/* Replaces khq_state_slot (src/csrc/qmv_sm75_kernel.cu:3968-3972; bound at src/ops.mojo:1025-1040):
 * address of one of three static void* cells the host parks module state in; `which` outside
 * 0..2 is clamped to 0. */
void* khq_state_slot(int which);

/* Replaces launch_khq_compress_fp16 (src/csrc/qmv_sm75_kernel.cu:4279-4310; typedef
 * src/ops.mojo:1060-1073).  n rows of d==256 fp16 values -> KHQ code words.  is_v==0: writes
 * out_mask, out_norms, out_r_norms (residual scale), out_payload (40 B/row) and zeroes
 * out_shared_meta.  is_v==1: writes out_norms, out_r_norms (energy correction), out_payload
 * (104 B/row) and out_shared_meta (fp32 max residual); out_mask is not touched.
 * Returns -100 if n<=0 or d!=256.  Code words are bit-identical to the reference kernel's. */
int launch_khq_compress_fp16(const void* x, const void* d_vec, const void* rotor,
                             const void* centroids, const void* vq_centroids, void* out_mask,
                             void* out_norms, void* out_r_norms, void* out_payload,
                             void* out_shared_meta, int n, int d, float threshold_scale,
                             float alpha, int is_v, khq_stream_t stream);

/* Replaces launch_khq_attn_fp16 (src/csrc/qmv_sm75_kernel.cu:4314-4375; typedef
 * src/ops.mojo:1075-1098).  Attention of num_queries = num_heads*L_q query rows over c_len
 * compressed tokens, positions start_pos..start_pos+c_len-1.  Writes out_attn
 * (num_queries, D+2).  When num_splits>1, out_partial (num_queries, num_splits, D+2) receives
 * the per-split partials in the reference layout and is merged into out_attn.
 * stride_s is ignored.  Returns -100 if num_queries<=0 or c_len<=0, -101 if num_splits>1 and
 * out_partial is NULL, -103 for unsupported head shapes. */
int launch_khq_attn_fp16(const void* q, const void* k_payload, const void* v_payload,
                         const void* v_shared_meta, const void* k_mask, const void* k_norms,
                         const void* k_r_norms, const void* v_norms, const void* v_r_norms,
                         const void* centroids_k, const void* centroids_v,
                         const void* vq_centroids, const void* k_rotor, const void* v_rotor,
                         const void* d_vec_k, const void* d_vec_v, void* out_attn,
                         void* out_partial, int num_queries, int num_heads, int L_q, int c_len,
                         int stride_s, int n_rep, float scale, float alpha_k, float alpha_v,
                         float rope_base, int start_pos, int num_splits, khq_stream_t stream);

/* Replaces launch_khq_window_attn_fp16 (src/csrc/qmv_sm75_kernel.cu:4378-4396; typedef
 * src/ops.mojo:1181-1196).  Attention over win_len raw fp16 ring slots (win_start+s) % ring_cap;
 * ring rows are token-major (slot*H_kv + kv)*d; K is already RoPE'd.  Writes (H_q, D+2)
 * unnormalised.  Returns -100 if H_q<=0 or win_len<=0, -103 for unsupported shapes. */
int launch_khq_window_attn_fp16(const void* q, const void* ring_k, const void* ring_v,
                                void* out_attn, int win_start, int win_len, int ring_cap, int H_q,
                                int H_kv, int d, float scale, khq_stream_t stream);

/* Replaces launch_khq_merge_gate_fp16 (src/csrc/qmv_sm75_kernel.cu:4414-4429; typedef
 * src/ops.mojo:1245-1252).  LSE-merges the compressed and window partials when has_w!=0
 * (otherwise uses attn_c alone), divides by (den + 1e-8), multiplies by sigmoid(gate) and
 * writes fp16 (H_q, d).  Returns -100 if H_q<=0 or d<=0. */
int launch_khq_merge_gate_fp16(const void* attn_c, const void* attn_w, const void* q_gate,
                               void* out, int H_q, int d, int has_w, khq_stream_t stream);

/* Replaces launch_khq_gather_q_fp16 (src/csrc/qmv_sm75_kernel.cu:4399-4411): de-interleaves the
 * query half of q_gate into (H_q, d).  Used only by the reference's dump path. */
int launch_khq_gather_q_fp16(const void* q_gate, void* q_out, int H_q, int d,
                             khq_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Section 2: additions (no counterpart in the reference)
 * ---------------------------------------------------------------------------------------- */

/* ---- Batched decode: many (sequence, layer) problems in one persistent launch ------------ */

/* One decode problem: a sequence's KHQ state of one attention layer plus this step's query.
 * 128 bytes, device pointers, stored in a device-resident array. */
typedef struct khq_seq_desc {
    const void* q_gate;         /* (24, 512) fp16 */
    const void* k_payload;      /* compressed region, rows = token*4 + kv_head */
    const void* v_payload;
    const void* v_shared_meta;
    const void* k_mask;
    const void* k_norms;
    const void* k_r_norms;
    const void* v_norms;
    const void* v_r_norms;
    const void* ring_k;         /* (ring_cap, 4, 256) fp16, K already RoPE'd */
    const void* ring_v;
    void* out;                  /* (24, 256) fp16 gated attention output */
    int32_t table_id;           /* index into the khq_tables_desc array (the layer) */
    int32_t c_len;              /* compressed tokens */
    int32_t start_pos;          /* absolute position of compressed token 0 */
    int32_t win_start;          /* first ring slot of the raw window */
    int32_t win_len;            /* raw window tokens */
    int32_t first_slot;         /* filled by khq_b200_plan_decode */
    int32_t n_slots;            /* filled by khq_b200_plan_decode */
    int32_t pos_pack;           /* 0: compressed token s sits at position start_pos + s.  Otherwise the arrays
                                 * hold every G-th chunk of a longer context (chunk-cyclic context partition):
                                 * (pos_chunk << 16) | G, token s at start_pos + (s / pos_chunk) * G * pos_chunk
                                 * + s % pos_chunk; pos_chunk even.  Kernel generations 1 and 2 only (3 and 4 set
                                 * the device status word to 4). */
} khq_seq_desc;

/* One layer's calibration tables (fp16 device arrays in the khq_calib layout). 64 bytes. */
typedef struct khq_tables_desc {
    const void* cents_k;
    const void* cents_v;
    const void* vq;
    const void* k_rotor;
    const void* v_rotor;
    const void* d_k;
    const void* d_v;
    float alpha_k, alpha_v;
} khq_tables_desc;

/* One CTA-sized piece of a problem; produced by khq_b200_plan_decode. 32 bytes. */
typedef struct khq_work_item {
    int32_t desc, kind, lo, hi, slot, r0, r1, r2; /* kind 0: compressed tokens [lo,hi); 1: window */
} khq_work_item;

/* Host-side planner (pure CPU; its only CUDA call asks for the current device's SM count and falls
 * back to 148).  c_len[i]/win_len[i] describe problem i; problems should be ordered by table_id so
 * that consecutive items share tables.  The array order is the launch order (the CTAs pull items off
 * one counter): every raw window first, then the compressed regions in problem order, each cut into
 * pieces that start on even tokens.  Piece sizes: tokens_per_item tokens (rounded up to a multiple
 * of 96; <= 0 picks a size that fills the GPU) while more than 2 x SMs such pieces remain in the
 * launch, then remaining / (2 x SMs) down to 96 or 48 -- or, when that simulates shorter, one to three
 * equal pieces per SM.  Slots are numbered problem by problem (window first) whatever the array order.  Writes up to max_items items, and per problem the first partial slot
 * and the slot count (copy them into the descriptors).  Returns the item count (== total slot
 * count); a value > max_items means items_out was too small.  -100 on bad args. */
int khq_b200_plan_decode(const int* c_len, const int* win_len, int n_desc, int tokens_per_item,
                         void* items_out, int max_items, int* first_slot, int* n_slots);

/* Bytes of workspace launch_khq_decode_batched_fp16 needs for n_slots_total partial slots. */
size_t khq_b200_decode_workspace_bytes(int n_slots_total);

/* Whole decode attention (compressed region + raw window + LSE merge + sigmoid gate) of n_desc
 * problems: a persistent kernel (one CTA per SM pulling items off an atomic counter in the
 * workspace) followed by a merge kernel.  descs/tables/items are DEVICE arrays; workspace is a
 * 256-byte-aligned device buffer of at least khq_b200_decode_workspace_bytes(n_slots_total).
 * codebook_in_smem selects the kernel generation: 1 / 0 = CUDA-core kernel with each layer's V
 * codebook staged in shared memory / gathered from global memory, 2 = warp-level tensor-core kernel
 * (mma.sync), 3 = tcgen05 kernel (tensor-memory accumulators, code words decoded one payload row
 * per thread), 4 = the same formulation run by 32 light warps (two mask words or two patches per
 * thread, CTA-wide step barriers), -1 let the library choose.  Allocates nothing; the only non-kernel call is a 256-byte
 * cudaMemsetAsync on `stream`.  Returns -100 (empty/NULL arguments), -104 (alignment), -105
 * (workspace too small). */
int launch_khq_decode_batched_fp16(const void* descs, const void* tables, const void* items, int n_desc,
                                   int n_items, void* workspace, size_t workspace_bytes,
                                   int n_slots_total, float scale, float rope_base, int ring_cap,
                                   int codebook_in_smem, khq_stream_t stream);

/* The same launch ending in one unnormalised record (acc[256], max, sum_exp) per (problem, head),
 * out_partials (n_desc, 24, 258) fp32, instead of the gated fp16 outputs (khq_seq_desc::out is not
 * touched): the share of one GPU in a context-parallel step, merged across GPUs by
 * launch_khq_merge_slots_gate_fp16.  No counterpart in the reference (it serves one GPU).  Extra
 * returns: -100 (out_partials NULL), -104 (its alignment). */
int launch_khq_decode_batched_partial_fp16(const void* descs, const void* tables, const void* items, int n_desc,
                                           int n_items, void* workspace, size_t workspace_bytes,
                                           int n_slots_total, float scale, float rope_base, int ring_cap,
                                           int codebook_in_smem, void* out_partials, khq_stream_t stream);

/* ---- Pre-step: everything between the q/k/v projections and khq_step, in one launch --------
 * Replaces five launches of the reference host: head_rmsnorm_sm75_gpu on q and k
 * (src/models/qwen3_5/attention.mojo:329-336), khq_capture_unroped (src/khq/runtime.mojo:432-451),
 * partial_rope_sm75_gpu on q and k (attention.mojo:348-353) and the ring append of khq_step
 * (runtime.mojo:486).  In place: q_gate (H_q, 2*d) fp16 (query half normed + RoPE'd, gate half
 * untouched), k (H_kv, d) fp16 (normed + RoPE'd).  The three ring slot pointers address this
 * token's row of ring_u (K normed, un-RoPE'd), ring_k (K RoPE'd) and ring_v (V); any of them may
 * be NULL.  q_norm_w / k_norm_w: fp32 (d) or NULL.  The RMS normalisation always runs; has_norms == 0
 * (or a NULL weight) only drops the learned weight, as the reference's launcher does
 * (src/ops.mojo:1397-1411, the HAS_WEIGHT=False variant).  Half-split RoPE pairs (i, i + rotary_dim/2), freq = exp(log(theta) *
 * (-2i/rotary_dim)), fp32 angle pos*freq.  Returns -100 (bad arguments), -103 (shape), -104
 * (pointers not 16-byte aligned). */
int launch_khq_prestep_fp16(void* q_gate, void* k, const void* v, const void* q_norm_w,
                            const void* k_norm_w, void* ring_k_slot, void* ring_v_slot, void* ring_u_slot,
                            int H_q, int H_kv, int d, int rotary_dim, int pos, float rope_theta,
                            float rms_eps, int has_norms, khq_stream_t stream);

/* ---- The same pre-step for `batch` sequences in one launch (no counterpart in the reference, which
 * serves one sequence).  q_gate (batch, H_q, 2*d), k and v (batch, H_kv, d) fp16, in place as above.
 * ring_k / ring_v / ring_u: base of the first sequence's ring; sequence b's rings start
 * ring_seq_stride halfs further per b; its new token goes to slot slots[b] and is rotated at
 * position positions[b] (device int32 arrays of `batch` entries).  Same return codes. */
int launch_khq_prestep_batched_fp16(void* q_gate, void* k, const void* v, const void* q_norm_w,
                                    const void* k_norm_w, void* ring_k, void* ring_v, void* ring_u,
                                    long long ring_seq_stride, const void* slots, const void* positions,
                                    int batch, int H_q, int H_kv, int d, int rotary_dim, float rope_theta,
                                    float rms_eps, int has_norms, khq_stream_t stream);

/* ---- Many compression events in one launch (no counterpart in the reference).
 * launch_khq_compress_fp16 (src/csrc/qmv_sm75_kernel.cu:4279-4310) over `n_seg` runs of
 * `rows_per_seg` rows: run i reads its fp16 rows from segs[i].x + x_byte_offset and writes rows
 * segs[i].row0 .. segs[i].row0 + rows_per_seg - 1 of the output arrays.  `segs` is a device array
 * of khq_compress_seg.  Row by row the arithmetic and the code words are those of the single
 * launch.  Returns -100 (bad arguments), -104 (x_byte_offset not a multiple of 16). */
typedef struct khq_compress_seg {
    const void* x;      /* first source row of the run (fp16, d per row, contiguous) */
    long long row0;     /* first output row of the run */
} khq_compress_seg;
int launch_khq_compress_batched_fp16(const void* segs, int n_seg, int rows_per_seg, const void* d_vec,
                                     const void* rotor, const void* centroids, const void* vq_centroids,
                                     void* out_mask, void* out_norms, void* out_r_norms, void* out_payload,
                                     void* out_shared_meta, int d, float threshold_scale, float alpha,
                                     int is_v, long long x_byte_offset, khq_stream_t stream);

/* ---- Step-dependent descriptor fields of a batch engine (no counterpart in the reference).
 * `descs`: n_layers * n_seq khq_seq_desc, layer-major; `dyn`: n_seq khq_seq_dyn, the state that
 * moves every step and is the same for all layers of a sequence.  One launch copies dyn[s] into
 * the eight ints of descs[l * n_seq + s] for every layer l; the pointers stay.  Returns -100. */
typedef struct khq_seq_dyn {
    int c_len, start_pos, win_start, win_len, first_slot, n_slots, reserved0, reserved1;
} khq_seq_dyn;
int launch_khq_update_descs(void* descs, const void* dyn, int n_seq, int n_layers, khq_stream_t stream);

/* ---- One decode step of one sequence in two or three launches ------------------------------
 * What khq_step does between two compression events (src/khq/runtime.mojo:503-612: three ring
 * appends, launch_khq_attn_fp16 (+ its split reduce), launch_khq_window_attn_fp16,
 * launch_khq_merge_gate_fp16: seven launches there) as one call: the compressed-region attention over
 * c_len tokens with `num_splits` splits (skipped when c_len == 0; attn_c (24, 258) fp32 and
 * attn_partial (24, num_splits, 258) fp32 are the caller's scratch), then ONE kernel that appends
 * the step's token (k_roped, v_new, k_unroped: 4*256 halfs each; k_unroped / ring_u may be null) to
 * the rings at slot (win_start + win_len - 1) % ring_cap, runs the raw-window attention over the
 * win_len newest tokens (the step's own token included), merges with attn_c, divides by
 * (den + 1e-8), applies the sigmoid gate and writes out (24, 256) fp16.  Shapes are Bonsai-27B's
 * (24 / 4 heads, d 256).  Returns -100 (bad arguments), -103 (win_len > ring_cap), -104 (alignment)
 * or launch_khq_attn_fp16's codes. */
int launch_khq_decode_step_fp16(
    const void* q_gate, const void* k_roped, const void* v_new, const void* k_unroped, void* ring_k, void* ring_v,
    void* ring_u, const void* k_payload, const void* v_payload, const void* v_shared_meta, const void* k_mask,
    const void* k_norms, const void* k_r_norms, const void* v_norms, const void* v_r_norms, const void* centroids_k,
    const void* centroids_v, const void* vq_centroids, const void* k_rotor, const void* v_rotor, const void* d_vec_k,
    const void* d_vec_v, void* attn_c, void* attn_partial, void* out, int c_len, int win_start, int win_len, int ring_cap,
    int num_splits, float scale, float alpha_k, float alpha_v, float rope_base, khq_stream_t stream);

/* ---- Prefill: causal GQA attention + sigmoid gate over a whole prompt --------------------
 * The math of the reference's fp16-KV attention kernel (gqa_attention_sm75_gpu,
 * src/kernels/elementwise_sm75.mojo:1091-1231), which the reference launches once per prompt
 * token (src/models/qwen3_5/layer.mojo:630-641), for all T rows of `batch` prompts at once:
 *   out[b,t,h,:] = softmax_{u<=t}(q[b,t,h] . K[b,u,h/6] * scale) V[b,u,h/6] * sigmoid(gate[b,t,h,:])
 * with the kernel's 1/(Z + 1e-9) denominator.  q_gate (batch, T, H_q, 2*d) fp16 (query | gate
 * per head, the reference's interleaved layout), k / v (batch, T, H_kv, d) fp16 token-major (the
 * reference's KV-cache row layout), K already RoPE'd; out (batch, T, H_q, d) fp16.  Batch strides
 * are in elements.  Returns -100 (empty), -103 (d != 256 or H_q % H_kv != 0), -104 (pointers not
 * 16-byte aligned). */
int launch_khq_gqa_prefill_fp16(const void* q_gate, const void* k, const void* v, void* out, int batch,
                                int T, int H_q, int H_kv, int d, float scale, long long q_batch_stride,
                                long long kv_batch_stride, long long out_batch_stride,
                                khq_stream_t stream);

/* The two kernels behind launch_khq_gqa_prefill_fp16, with its arguments and error codes.  No
 * reference counterpart (the reference has one attention kernel, launched per token).
 *   _tc5_: tcgen05.mma with accumulators in tensor memory, operands staged by TMA tensor maps
 *          built per call; also returns -107 (the driver exposes no tensor-map encoder) or -108
 *          (the encoder refused the shapes; batch strides must be multiples of 8 elements).
 *   _mma_: warp-level mma.sync kernel.
 * khq_b200_prefill_select(0) routes launch_khq_gqa_prefill_fp16 to _tc5_ (the default), (1) to
 * _mma_; returns -100 for any other value.  khq_b200_prefill_status() synchronises the device,
 * returns and clears the _tc5_ kernel's status word: 0 clean, 1 a bounded wait ran out (the
 * output of that launch is then meaningless), -1 the read failed. */
int launch_khq_gqa_prefill_tc5_fp16(const void* q_gate, const void* k, const void* v, void* out, int batch,
                                    int T, int H_q, int H_kv, int d, float scale, long long q_batch_stride,
                                    long long kv_batch_stride, long long out_batch_stride,
                                    khq_stream_t stream);
int launch_khq_gqa_prefill_mma_fp16(const void* q_gate, const void* k, const void* v, void* out, int batch,
                                    int T, int H_q, int H_kv, int d, float scale, long long q_batch_stride,
                                    long long kv_batch_stride, long long out_batch_stride,
                                    khq_stream_t stream);
/* The same attention over bf16 tensors (bf16 operands and probabilities, fp32 accumulation, bf16
 * output): the _tc5_ kernel with its bf16 instruction format.  Same arguments, layouts and error
 * codes as launch_khq_gqa_prefill_tc5_fp16.  No reference counterpart (the reference is fp16 only). */
int launch_khq_gqa_prefill_bf16(const void* q_gate, const void* k, const void* v, void* out, int batch, int T,
                                int H_q, int H_kv, int d, float scale, long long q_batch_stride,
                                long long kv_batch_stride, long long out_batch_stride, khq_stream_t stream);
int khq_b200_prefill_select(int which);
/* Work distribution of the _tc5_ kernel: 0 = by prompt length (persistent CTAs up to 24 row blocks of
 * 128 rows, one CTA per 128-row item beyond), 1 = one item per CTA, n > 1 = n items per CTA (a large
 * n gives one persistent CTA per SM).  Returns -100 for a negative n. */
int khq_b200_prefill_tc5_items_per_cta(int n);
int khq_b200_prefill_status(void);

/* ---- Context parallelism: one long sequence split by context range over several GPUs ------
 * Each GPU calls launch_khq_attn_fp16 on its slice (start_pos = first absolute token of the
 * slice) and obtains an unnormalised (24, 258) partial; the owner of the raw ring adds the
 * window partial.  After the partials have been gathered slot-major, (n_slots, 24, 258) fp32,
 * this launch LSE-merges them, divides by (den + 1e-8), applies the sigmoid gate and writes
 * fp16 (24, 256): the math of khq_attn_reduce_kernel + khq_merge_gate_kernel
 * (src/csrc/qmv_sm75_kernel.cu:1836-1877, 1983-2010) over n_slots regions.  Slots that hold
 * (0, -1e20, 0) are neutral.  Returns -100 (bad arguments), -103 (shape). */
int launch_khq_merge_slots_gate_fp16(const void* partials, int n_slots, const void* q_gate, void* out,
                                     int H_q, int d, khq_stream_t stream);

/* No counterpart in the reference (it serves one GPU).  launch_khq_attn_fp16 over a slice that holds
 * every G-th `pos_chunk`-token chunk of a longer context, which is what a GPU holds when the
 * compressed region is partitioned chunk-cyclically over G GPUs (chunk c on GPU c mod G, so appended
 * chunks keep the GPUs balanced): token s of the arrays sits at absolute position
 * start_pos + (s / pos_chunk) * pos_stride + s % pos_chunk (GPU g of G: start_pos = g * 128,
 * pos_chunk = 128, pos_stride = G * 128).  Same arguments otherwise, without `stride_s`.  pos_chunk
 * must be positive and even, pos_stride >= pos_chunk, else -103. */
int launch_khq_attn_strided_fp16(const void* q, const void* k_payload, const void* v_payload,
                                 const void* v_shared_meta, const void* k_mask, const void* k_norms,
                                 const void* k_r_norms, const void* v_norms, const void* v_r_norms,
                                 const void* centroids_k, const void* centroids_v,
                                 const void* vq_centroids, const void* k_rotor, const void* v_rotor,
                                 const void* d_vec_k, const void* d_vec_v, void* out_attn, void* out_partial,
                                 int num_queries, int num_heads, int L_q, int c_len, int n_rep, float scale,
                                 float alpha_k, float alpha_v, float rope_base, int start_pos, int num_splits,
                                 int pos_chunk, int pos_stride, khq_stream_t stream);

/* No counterpart in the reference.  launch_khq_attn_fp16 for callers that cannot hand over a
 * partial buffer: the split partials go to a fixed array inside the library's device image
 * (24 heads x up to 32 splits x 258 floats = 792 576 bytes per GPU that loads the library)
 * instead of `out_partial`.  Meant for hosts whose device memory is entirely owned by another
 * runtime's pool, or that sit inside a decode loop where cudaMalloc (which synchronises the
 * whole device) is not acceptable.  Same arguments and results as launch_khq_attn_fp16 without
 * `out_partial` and `stride_s`; restricted to L_q == 1, num_queries == 24, num_splits <= 32,
 * anything larger returns -106.  It calls no allocating routine.  The first call on a device
 * looks up the array's device address (cudaGetSymbolAddress) and caches it, so make that first
 * call outside any stream capture, and from one host thread (the per-device caches are plain
 * statics: first calls racing from several host threads on one device are not supported).  Every call on a device shares the one array: calls that may
 * overlap on the GPU (different streams) race on it; calls on one stream do not.  Nothing in the
 * array has to be cleared between calls: every split writes its whole record, empty splits
 * included. */
int launch_khq_attn_static_fp16(const void* q, const void* k_payload, const void* v_payload,
                                const void* v_shared_meta, const void* k_mask, const void* k_norms,
                                const void* k_r_norms, const void* v_norms, const void* v_r_norms,
                                const void* centroids_k, const void* centroids_v,
                                const void* vq_centroids, const void* k_rotor, const void* v_rotor,
                                const void* d_vec_k, const void* d_vec_v, void* out_attn,
                                int num_queries, int num_heads, int L_q, int c_len, int n_rep,
                                float scale, float alpha_k, float alpha_v, float rope_base,
                                int start_pos, int num_splits, khq_stream_t stream);

/* ---- Calibration: the K-static fit -----------------------------------------------------------
 * cal_kstatic_p_kernel + cal_kstatic_f_kernel of the reference (src/csrc/qmv_sm75_kernel.cu:2645-2680;
 * op 2 of launch_cal_op, :4634-4643): from the projected K sample `rot` (rows, 256) fp32 the per-dim
 * sigma, the threshold scale ts = 16 / sqrt(sum_i 0.528756 (0.935 sigma_i)^2 + 0.464545 sigma_i^2)
 * and the four base centroid rows {0, -cb, +cb, +cb}, cb_i = 0.935 sigma_i ts (`cents`, 4 x 256 fp32;
 * `out_ts`, 1 fp32; `sigma_out`, 256 fp32 or NULL; all device memory).  Same summation order as the
 * reference, so the tables are bit-identical; unlike it, nothing is allocated and the stream is not
 * synchronised.  The other calibration operations are offline work outside this library.
 * Returns -100 on bad arguments. */
int launch_khq_cal_kstatic_fp32(const void* rot, int rows, void* cents, void* out_ts, void* sigma_out,
                                khq_stream_t stream);

/* Library identification: "khq-b200 <version> sm_100a". */
const char* khq_b200_version(void);

/* Word written by the decode kernels when a bounded wait on an asynchronous copy gave up
 * (0 = never).  Reads the device flag of the current device with a blocking 4-byte copy, so
 * call it outside the hot loop.  Returns the flag, or -(cudaError_t) on failure. */
int khq_b200_device_status(void);
/* The same read, then the word is reset to 0.  Values: 1 = a bounded wait on an asynchronous copy
 * gave up, 2 = a tensor-core decode kernel found its shared memory misaligned, 3 =
 * launch_khq_merge_slots_wait_gate_fp16 gave up waiting for a peer's flag, 4 = a descriptor asked a
 * decode kernel generation for chunk-cyclic positions it does not support. */
int khq_b200_device_status_clear(void);

/* ---- Context parallelism without a collective library: partials exchanged over peer memory ----
 * Every GPU owns a slot buffer (2 parities x n_slots records of 24 x 258 floats) and a flag array
 * (one 32-bit word per producer GPU), both mapped into the other processes (CUDA IPC).
 * launch_khq_publish_partials_fp32 copies `n_records` consecutive (24, 258) records from `src` into
 * slots first_slot.. of EVERY peer's buffer (peer_slots / peer_flags: device arrays of `world`
 * pointers, entry p = GPU p's buffer as mapped here; parity_offset_records selects the parity
 * half), fences system-wide and stores `epoch` into flag[rank] of every peer: one CTA per peer,
 * plain stores over NVLink.  launch_khq_merge_slots_wait_gate_fp16 is
 * launch_khq_merge_slots_gate_fp16 preceded by a wait for flags[0..n_flags) >= epoch (modulo
 * 2^32), bounded by `max_polls` polls of ~64 ns (0 = 2^22): when it runs out the status word
 * becomes 3 and the launch still completes.  Epochs grow by one per step; a producer is at most one
 * step ahead of a consumer, so two parities of slots suffice.  No reference counterpart.
 * Return -100 (bad arguments), -103 (shape), -104 (alignment). */
/* Enables peer access from the current device to `peer_device` (a CUDA IPC mapping of a peer's
 * buffer lives in the peer's context; kernels of the current device may dereference it only after
 * this).  0 = enabled (or already enabled, or the same device), -109 = the GPUs are not peers. */
int khq_b200_enable_peer_access(int peer_device);
/* Peer-visible buffers for that exchange.  khq_b200_peer_alloc: cudaMalloc + zero fill on the current
 * device, returns the pointer and the 64-byte CUDA IPC handle of the allocation (to be sent to the
 * other processes).  khq_b200_peer_open: maps another process's allocation for the current device
 * (the open enables peer access between the two GPUs).  khq_b200_peer_close / _free undo them.
 * khq_b200_peer_poke / _peek: blocking 4-byte write / read through the runtime, with which a host
 * checks a mapping before any kernel uses it.  All return 0, a positive cudaError_t, or -100. */
int khq_b200_peer_alloc(size_t bytes, void** ptr_out, unsigned char* handle_out);
int khq_b200_peer_open(const unsigned char* handle, void** ptr_out);
int khq_b200_peer_close(void* ptr);
int khq_b200_peer_free(void* ptr);
int khq_b200_peer_poke(void* dst, unsigned int value);
int khq_b200_peer_peek(const void* src, unsigned int* value_out);
int launch_khq_publish_partials_fp32(const void* src, int n_records, const void* peer_slots, const void* peer_flags,
                                     int world, int rank, int first_slot, long long parity_offset_records,
                                     unsigned int epoch, khq_stream_t stream);
/* launch_khq_publish_bytes: the same publish for any payload (here: the owner's q_gate): `bytes`
 * (multiple of 16) from `src` to byte offset dst_byte_offset of every peer's buffer (peer_bufs:
 * device array of `world` base pointers), then `epoch` into word flag_index of every peer's flag
 * array.  launch_khq_wait_flag: a one-thread kernel that waits (bounded as above) until
 * *flag >= epoch, so that the kernels queued behind it on the stream see the payload.
 * Return -100 (bad arguments), -104 (alignment). */
int launch_khq_publish_bytes(const void* src, size_t bytes, const void* peer_bufs, long long dst_byte_offset,
                             const void* peer_flags, int flag_index, int world, unsigned int epoch, khq_stream_t stream);
int launch_khq_wait_flag(const void* flag, unsigned int epoch, unsigned int max_polls, khq_stream_t stream);
int launch_khq_merge_slots_wait_gate_fp16(const void* partials, const void* flags, int n_flags, unsigned int epoch,
                                          int n_slots, const void* q_gate, void* out, int H_q, int d,
                                          unsigned int max_polls, khq_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* KHQ_B200_H_ */
