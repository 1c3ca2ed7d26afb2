/* fast_mimi_b200 — C ABI of the B200 (sm_100a) kernels for Mimi's transformer self-attention.
 *
 * Conventions (the reference's own native-launcher convention: `extern "C" int fn(void* ptrs...,
 * int dims..., void* stream)`, e.g. src/fast_mimi/_native_cutlass.py:110-116 binding
 * src/fast_mimi/cutlass_bias_dgrad.cu:147-157):
 *   - every pointer is a raw DEVICE pointer owned by the caller; nothing is allocated or freed here;
 *   - `stream` is a cudaStream_t (0 = legacy default stream); launches are asynchronous on it;
 *   - the return value is 0 on success, a positive cudaError_t / CUresult, or a negative code for a
 *     rejected geometry (-1 bad size, -3 misaligned pointer, -4 driver entry point unavailable);
 *   - `status` (optional, may be NULL) is a caller-zeroed device int; a kernel whose bounded wait on
 *     a TMA / tensor-core completion barrier runs out writes a code >= 101 there and finishes early.
 *     Read it back with fm_read_status().
 *   - geometry of the tensor-core entry points is Mimi's: hidden 512, 8 heads of 64.
 *   - value_dtype: bit 0 selects the storage type of V, of the softmax probabilities fed to the tensor
 *     core and of the prefill output: 0 = BF16, 1 = FP16.  Q and K are always BF16.  In the entry points
 *     that contain the projection, bit 1 (value 2) says that x and w_qkv hold FP16 instead of BF16 (same
 *     tensor-core rate, 8x finer rounding of FP32 activations and weights; needs |values| < 65504).
 *
 * Tensors named "frames" are [B, T, 512] row-major (heads are 64-column slices), which is the
 * memory layout behind the reference's [B, 8, T, 64] strided views (src/fast_mimi/model.py:1897-1911).
 */
#ifndef FAST_MIMI_B200_H_
#define FAST_MIMI_B200_H_

#ifdef __cplusplus
extern "C" {
#endif

int fm_abi_version(void);

/* Self-test of the bounded device waits every kernel of this library uses (no counterpart in the reference, whose
 * kernels do not wait on one another): a one-thread kernel waits, with a limit of limit_us microseconds (at most
 * 100 000), on a barrier that nothing arrives on.  The wait gives up, code 103 lands in *status and the kernel
 * returns normally.  observed (3 ints, may be NULL): whether the first wait succeeded (0 expected), whether a second
 * wait in the same block succeeded (0), whether that second wait returned at once because the block was already
 * marked aborted (1). */
int fm_selftest_wait_timeout(int* status, int limit_us, int* observed, void* stream);

/* q|k|v = x W_qkv^T with rotate-half RoPE applied to q and k in the FP32 epilogue.
 * Replaces q_proj/k_proj/v_proj + _apply_rope (src/fast_mimi/model.py:1897-1912; packed-weight form
 * src/fast_mimi/_packed_qkv.py:139-171).
 *   x      [B*T, 512] BF16          w_qkv [1536, 512] BF16 = cat(Wq, Wk, Wv) rows
 *   cos,sin [1 or B, T, 64] FP32 (the reference's position_embeddings); cos_bstride = 0 or T*64.
 *           Columns 32..63 repeat columns 0..31 (MimiRotaryEmbedding builds them so,
 *           src/fast_mimi/model.py:1533); the kernel reads the first 32.
 *   q,k    [B*T, 512] BF16 out      v [B*T, 512] value_dtype out */
int fm_qkv_rope_bf16(const void* x, const void* w_qkv, const float* cos, const float* sin,
                     long long cos_bstride, void* q, void* k, void* v, int B, int T, int value_dtype,
                     int* status, void* stream);

/* Banded causal attention over already-rotated q, k: key j visible to query i iff i-window < j <= i.
 * Replaces _sdpa_fallback's masked SDPA (src/fast_mimi/model.py:1823-1868, mask :1672-1676) and
 * _native_window_attention (src/fast_mimi/model.py:1589-1624).
 *   q,k [B, T, 512] BF16; v, out [B, T, 512] value_dtype.  scale is applied to q.k (0.125 for Mimi). */
int fm_band_attn_prefill_bf16(const void* q, const void* k, const void* v, void* out, int B, int T,
                              int window, float scale, int value_dtype, int* status, void* stream);

/* Banded attention of Tq query frames against Tk >= Tq key / value frames whose last Tq rows are the queries' own
 * frames and whose first Tk - Tq rows are older (cached) frames: the masked SDPA of a cached call with
 * query_offset - key_offset = Tk - Tq (src/fast_mimi/model.py:1672-1677, :2194-2205) on rotated q [B,Tq,512] BF16,
 * k [B,Tk,512] BF16, v [B,Tk,512] (value type) -> out [B,Tq,512].  Tk == Tq is fm_band_attn_prefill_bf16. */
int fm_band_attn_chunk_bf16(const void* q, const void* k, const void* v, void* out, int B, int Tq, int Tk, int window,
                            float scale, int value_dtype, int* status, void* stream);

/* The same computation as fm_attention_prefill_bf16 in ONE kernel for clips of 128 < T <= 256 frames (Mimi's
 * 10 s clips): x and W_qkv in, attention output out, the rotated q, k, v never reach memory, so no workspace.
 * Replaces src/fast_mimi/model.py:1897-1914 + :1627-1688 + :1860-1868 for such clips (the reference's own fused
 * front half: src/fast_mimi/_packed_qkv.py:14-131,152-202).  Other T: returns -6 (use fm_attention_prefill_bf16).
 * It moves 2.5 times fewer bytes through HBM than the two kernels and is the faster of the two forms on B200;
 * fm_attention_prefill_bf16 routes such clips to it.  value_dtype as for
 * fm_qkv_rope_bf16. */
int fm_attention_fused_bf16(const void* x, const void* w_qkv, const float* cos, const float* sin, long long cos_bstride,
                            void* out, int B, int T, int window, float scale, int value_dtype, int* status,
                            void* stream);

/* A call with T >= 1 new frames per stream on top of a KV ring that already holds `past` frames: the cached
 * multi-frame call of the reference (chunked streaming encode: MimiAttention.forward with q_len > 1 and a cache,
 * src/fast_mimi/model.py:1912-1914; keys = the last window-1 cached rows + the new rows, MimiKVCache.update
 * src/fast_mimi/model.py:450-471; band with query_offset = past, key_offset = max(past - (window-1), 0),
 * src/fast_mimi/model.py:2194-2205, :1672-1677).  Projection + RoPE into q_ws / k_ws / v_ws [S, T, 512]; when
 * past > 0 the still-visible ring rows and the new rows are laid out frame-major in k_lin / v_lin
 * [S, min(past, window-1) + T, 512] (may be NULL when past == 0); banded attention writes out [S, T, 512]
 * (value type); finally the newest min(T, ring_slots) new rows enter the ring [S, 8, ring_slots, 64] at slot
 * position % ring_slots.  cos / sin are the tables of positions past .. past+T-1.  ring_slots >= window. */
int fm_attention_chunk_bf16(const void* x, const void* w_qkv, const float* cos, const float* sin, long long cos_bstride,
                            void* q_ws, void* k_ws, void* v_ws, void* k_lin, void* v_lin, void* ring_k, void* ring_v,
                            void* out, int S, int T, int past, int ring_slots, int window, float scale, int value_dtype,
                            int* status, void* stream);

/* y = residual + layer_scale * (attn W_o^T): the output projection that follows the attention core
 * (src/fast_mimi/model.py:1961) with the layer scale and residual add of the transformer layer
 * (src/fast_mimi/model.py:2059) folded into the FP32 epilogue.  Same persistent tensor-core kernel as
 * fm_qkv_rope_bf16, run over the two 256-wide output tiles of W_o.
 *   attn  [frames, 512], w_o [512, 512]: BF16, or FP16 when value_dtype bit 1 is set
 *   y, residual [frames, 512]: BF16, or FP16 when value_dtype bit 0 is set; residual may be NULL, and may
 *           alias y (each element is read by the thread that then writes it)
 *   layer_scale [512] FP32 or NULL (no scaling) */
int fm_out_proj_f16(const void* attn, const void* w_o, const float* layer_scale, const void* residual, void* y,
                    long long frames, int value_dtype, int* status, void* stream);

/* General bias-free linear layer with a fused epilogue on the tensor core:
 *   y = residual + scale * act(a W^T),  act = identity (activation 0) or exact erf GELU (activation 1).
 * Replaces the MLP's fc1 + GELU and fc2 + layer scale + residual add (src/fast_mimi/model.py:1990-1999,
 * :2060-2061) and, for FP32 residual streams, o_proj + layer scale + residual (src/fast_mimi/model.py:1961, :2059).
 *   a [rows, k_in], w [n_out, k_in]: in_dtype 0 = BF16, 1 = FP16.  k_in a multiple of 64, n_out of 256.
 *   y, residual [rows, n_out]: out_dtype 0 = BF16, 1 = FP16, 2 = FP32; residual may be NULL or alias y.
 *   scale [n_out] FP32 or NULL. */
int fm_linear_f16(const void* a, const void* w, const float* scale, const void* residual, void* y,
                  long long rows, int n_out, int k_in, int in_dtype, int out_dtype, int activation,
                  int* status, void* stream);

/* LayerNorm over the 512 channels of each frame, FP32 arithmetic, biased variance (nn.LayerNorm as used in
 * src/fast_mimi/model.py:2021-2024, :2052, :2060), with the result rounded once to the 16-bit type the
 * projections consume.
 *   x [rows, 512]: x_dtype 0 = BF16, 1 = FP16, 2 = FP32     y [rows, 512]: y_dtype 0 = BF16, 1 = FP16
 *   weight, bias [512] FP32 */
int fm_layernorm_f16(const void* x, int x_dtype, const float* weight, const float* bias, float eps, void* y,
                     int y_dtype, long long rows, void* stream);

/* One layer of residual vector quantisation for `rows` frames of 256 dimensions against a codebook of n_codes
 * entries: replaces MimiEuclideanCodebook.quantize (argmin over torch.cdist, src/fast_mimi/model.py:2277-2291) and
 * the residual update of MimiResidualVectorQuantizer.encode (src/fast_mimi/model.py:2420-2427).
 *   scores    [rows, n_codes], scores_dtype 1 = FP16 or 2 = FP32 (the out_dtype codes of fm_linear_f16): inner
 *             products residual . e_j computed from FP16 copies of both (fm_linear_f16 with a = residual16,
 *             w = FP16 codebook); they pre-select only
 *   e_sq      [n_codes] FP32: |e_j|^2      codebook [n_codes, 256] FP32      e_max = max_j |e_j|
 *   residual  [rows, 256] FP32, in/out: the chosen entry is subtracted
 *   residual16 [rows, 256] FP16 out: copy of the new residual for the next layer's inner products
 *   codes     [rows] int64 out        n_candidates [rows] int32 out or NULL (entries that were decided exactly)
 * Every entry whose approximate distance is within tau_rel * |residual| * e_max of the minimum is re-evaluated as
 * sum_k (x_k - e_jk)^2 in FP32; the smallest wins, the lowest index on ties.  tau_rel = 4.5e-3 covers the FP16
 * operand rounding with FP32 scores, 6.0e-3 with FP16 scores (twice the worst-case error of a distance).
 * A frame whose residual is not finite has no candidate: code 105 is recorded in *status (NULL = not recorded). */
int fm_rvq_select_f32(const void* scores, int scores_dtype, const float* e_sq, const float* codebook,
                      float* residual, void* residual16, long long* codes, int* n_candidates, long long rows,
                      int n_codes, float e_max, float tau_rel, int* status, void* stream);

/* Input rows of the stride-2 downsampling convolution that follows the encoder transformer (MimiModel.downsample:
 * MimiConv1d(512, 512, kernel 4, stride 2, no bias, replicate padding, causal), src/fast_mimi/model.py:2734-2744):
 * for frame-major FP32 x [B, T, C], row (b, t) of the result is frames stride*t - (kernel - stride) .. + kernel - 1
 * of clip b, clamped to the clip (replicate padding on both sides), C values each, as FP16 hi + lo parts
 * [B * ceil(T / stride), kernel * C].  The convolution itself is then fm_linear_f16 with the kernel laid out as
 * [C_out, kernel * C_in] (three products: hi W_hi + hi W_lo + lo W_hi, FP32 residual chaining). */
int fm_conv_rows_split(const float* x, void* hi, void* lo, int B, int T, int C, int kernel, int stride, void* stream);

/* The stride-2 upsampling that precedes the decoder transformer (MimiModel.upsample: MimiConvTranspose1d(512, 512,
 * kernel 4, stride 2, groups 512, no bias), src/fast_mimi/model.py:2745-2753; its forward trims the last two output
 * frames): x [B, T, C] FP32 frame-major, w [C, 4] FP32 (the ConvTranspose1d weight [C, 1, 4]) -> y [B, 2T, C] FP32,
 * y[b, n, c] = w[c, n % 2] x[b, n / 2, c] + w[c, n % 2 + 2] x[b, n / 2 - 1, c]. */
int fm_upsample2_f32(const float* x, const float* w, float* y, int B, int T, int C, void* stream);

/* x = hi + lo, both FP16 (hi = round(x), lo = round(x - hi)), n a multiple of 8 values: the operands of an
 * FP32-grade product on the FP16 tensor core (hi W_hi + hi W_lo + lo W_hi via fm_linear_f16 with FP32 residual
 * chaining).  Used for the quantiser's 1 x 1 input / output projections (nn.Conv1d(kernel 1, no bias),
 * src/fast_mimi/model.py:2392-2406, applied at :2417 and :2443), whose results decide code indices and must
 * therefore keep FP32 accuracy. */
int fm_split_half(const float* x, void* hi, void* lo, long long n, void* stream);

/* The same layer without the scores' round trip through memory (replaces the same reference lines as
 * fm_rvq_select_f32: src/fast_mimi/model.py:2277-2291, :2420-2427), three calls:
 *   fm_rvq_prepare_f32     before the first layer: FP16 copy of x [rows, 256] and every frame's candidate margin
 *                          tau[row] = tau_rel * |x| * e_max + 3.1e-5 * e_max (e_max of the FIRST layer's codebook)
 *   fm_rvq_candidates_f16  the inner products residual16 [rows, 256] x codebook16 [n_codes, 256]^T on the tensor core
 *                          (FP16 operands); the epilogue turns every 64 of them into one 16-byte record {minimum of
 *                          d_j = e_sq[j] - 2 x.e_j, 64-bit mask of the entries with d_j <= minimum + tau[row]}:
 *                          records [rows, n_codes / 64] x 16 B; n_codes a multiple of 256, at most 2048
 *   fm_rvq_select_rec_f32  exact FP32 decision among the entries flagged in the groups whose minimum is within tau of
 *                          the frame's global minimum (lowest index on ties), residual update, FP16 copy, and the
 *                          frame's margin for the NEXT layer (e_max_next = that layer's max |e_j|; 0 after the last)
 * With FP32 accumulation in the GEMM and no FP16 storage of the scores, tau_rel = 4.5e-3 covers the operand rounding. */
int fm_rvq_prepare_f32(const float* x, void* residual16, float* tau, long long rows, float e_max, float tau_rel,
                       void* stream);
int fm_rvq_candidates_f16(const void* residual16, const void* codebook16, const float* e_sq, const float* tau,
                          void* records, long long rows, int n_codes, int* status, void* stream);
int fm_rvq_select_rec_f32(const void* records, const float* codebook, float* residual, void* residual16, long long* codes,
                          int* n_candidates, float* tau, long long rows, int n_codes, float e_max_next, float tau_rel,
                          int* status, void* stream);

/* FP16 copy of [rows, 256] FP32 values (the residual before the first layer). */
int fm_rvq_to_half(const float* x, void* y, long long rows, void* stream);

/* out[row] = ((0 + E_0[codes[0,row]]) + E_1[codes[1,row]]) + ... in FP32, layers left to right, as
 * MimiResidualVectorQuantizer.decode does before output_proj (src/fast_mimi/model.py:2431-2444).
 *   codes [n_layers, rows] int64      codebooks [n_layers, n_codes, 256] FP32      out [rows, 256] FP32
 *   bad_code: optional device int set to 1 when an index is out of range (that index is then read as 0). */
int fm_rvq_decode_f32(const long long* codes, const float* codebooks, float* out, long long rows, int n_layers,
                      int n_codes, int* bad_code, void* stream);

/* The part of MimiAttention.forward between the input and o_proj (src/fast_mimi/model.py:1896-1951) for a call
 * without cache: fm_attention_fused_bf16 for clips of 128 < T <= 256 frames, else fm_qkv_rope_bf16 followed by
 * fm_band_attn_prefill_bf16 on the same stream.  q_ws/k_ws/v_ws are caller-provided workspaces of B*T*512 16-bit
 * elements each for the two-kernel form (not touched, and allowed to be null, when 128 < T <= 256). */
int fm_attention_prefill_bf16(const void* x, const void* w_qkv, const float* cos, const float* sin,
                              long long cos_bstride, void* q_ws, void* k_ws, void* v_ws, void* out, int B,
                              int T, int window, float scale, int value_dtype, int* status, void* stream);

/* Same computation as fm_attention_prefill_bf16 for callers that cannot hand over workspaces.
 * (No counterpart in the reference, whose launchers always receive caller-allocated buffers.)
 * Some hosts of this library may not call cudaMalloc at all: an allocation-free real-time audio loop
 * (an allocation can stall for milliseconds and drop frames), plugins whose host application owns every
 * device allocation, processes that budgeted their device memory up front.  For them the rotated q, k, v go to a
 * workspace that is part of the library image: a file-scope __device__ array of
 * FM_STATIC_MAX_FRAMES (8192) frames = 24 MiB, present on every GPU that loads the library until the
 * process exits.  The call allocates nothing and frees nothing.
 *   - B*T above FM_STATIC_MAX_FRAMES is rejected with -5 before anything is launched.
 *   - The first call on each device looks the workspace address up (one host-side runtime query, no
 *     launch); make that first call before starting any stream capture.
 *   - All calls share the one workspace and it keeps the previous call's contents.  Nothing in it needs
 *     to start at zero: the projection overwrites every frame row that the attention then reads.  Two
 *     calls whose kernels can overlap on the GPU (different streams, or the same stream from different
 *     threads without ordering) race on it; serialise them.
 * x, w_qkv, cos, sin, out, status, stream: as fm_attention_prefill_bf16. */
#define FM_STATIC_MAX_FRAMES 8192
int fm_attention_prefill_static_bf16(const void* x, const void* w_qkv, const float* cos, const float* sin,
                                     long long cos_bstride, void* out, int B, int T, int window, float scale,
                                     int value_dtype, int* status, void* stream);

/* One streaming step for S streams: project the new frame, rotate q/k at the stream's position,
 * write k/v into slot (position % ring_slots) of the stream's ring, attend over the valid slots.
 * Replaces MimiKVCache.update + one-query SDPA (src/fast_mimi/model.py:1912-1914, 435-471, 1860-1868).
 *   x [S, 512] BF16; cos,sin [1 or S, 1, 64] FP32 at each stream's position (cos_bstride 0 or 64)
 *   stream_pos: optional device int[S]; position of the new frame = pos_base + stream_pos[s]
 *   q_ws [S, 512] BF16 workspace; ring_k BF16 / ring_v value_dtype: [S, 8, ring_slots, 64]
 *   out [S, 512] FP32.  ring_slots = sliding window (250 for Mimi), at most 256. */
int fm_decode_step_bf16(const void* x, const void* w_qkv, const float* cos, const float* sin,
                        long long cos_bstride, const int* stream_pos, int pos_base, void* q_ws, void* ring_k,
                        void* ring_v, float* out, int S, int ring_slots, float scale, int value_dtype,
                        int* status, void* stream);

/* The attention half of the step alone (q and the ring already hold the new frame). */
int fm_ring_attn_decode_bf16(const void* q, const void* ring_k, const void* ring_v, float* out,
                             const int* stream_pos, int pos_base, int S, int ring_slots, float scale,
                             int value_dtype, int* status, void* stream);

/* FP32 verification path on CUDA cores, generic in heads / head_dim (<= 256) / window / offsets.
 * Same semantics as the eager branch of the reference (src/fast_mimi/model.py:1953-1958) with the
 * mask of _attention_mask at absolute positions (src/fast_mimi/model.py:1672-1676):
 * query i has position i+q_off, key j has position j+k_off.
 * strides[12] = {q_b,q_h,q_t, k_b,k_h,k_t, v_b,v_h,v_t, out_b,out_h,out_t} in elements; head_dim is
 * contiguous.  q, k already rotated. */
int fm_band_attn_fp32_verify(const float* q, const float* k, const float* v, float* out, int B, int H, int D,
                             int Tq, int Tk, int q_off, int k_off, int window, float scale,
                             const long long* strides, void* stream);

/* y[M,N] = x[M,K] w[N,K]^T in FP32 (F.linear without bias, src/fast_mimi/_functional_runtime.py:138-141). */
int fm_linear_fp32_verify(const float* x, const float* w, float* y, int M, int N, int K, void* stream);

/* In-place rotate-half RoPE on t [B, T, H, D] FP32 (src/fast_mimi/model.py:1538-1569). */
int fm_rope_fp32_verify(float* t, const float* cos, const float* sin, int B, int T, int H, int D,
                        long long cos_bstride, void* stream);

/* Synchronise `stream` and return the device status word (0 = all bounded waits completed). */
int fm_read_status(const int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FAST_MIMI_B200_H_ */
