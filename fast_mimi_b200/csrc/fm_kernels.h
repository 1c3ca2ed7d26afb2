// Internal launcher declarations shared by the .cu files of the library.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fm {

// Where the projection epilogue puts its results.  Linear outputs are [M, 512] 16-bit tensors
// (null = skip).  The KV ring is [clips, 8 heads, ring_slots, 64]; the frame at absolute position
// p of a clip lands in slot p % ring_slots.
struct QkvEpilogueArgs {
  uint16_t* q;
  uint16_t* k;
  uint16_t* v;
  uint16_t* ring_k;
  uint16_t* ring_v;
  const float* cos;        // [1 or clips, T, 64] FP32, as the reference's position_embeddings
  const float* sin;
  long long cos_bstride;   // 0 (one table for all clips) or T*64
  const int* clip_pos;     // optional device array: absolute position of frame 0 of each clip
  int pos_base;            // added to every position
  int T;                   // frames per clip in this call
  int ring_slots;
  // Output projection mode (launch_out_proj_gemm): the weight has two 256-wide output tiles instead of
  // six, results go out through `v` without RoPE as  resid + out_scale[c] * acc  (both optional).
  int n_tiles;             // 256-wide output tiles of the weight: 6 (q|k|v) or 2 (one 512-wide output)
  int seg_base;            // segment of output tile 0: 0 (q, k, v in turn) or 2 (plain output)
  const float* out_scale;  // [512] per-channel factor (the reference's layer scale) or null
  const uint16_t* resid;   // [M, 512] residual in the output's 16-bit format or null
};

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time libcuda).
int encode_tiled(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t rank, void* base, const cuuint64_t* dims,
                 const cuuint64_t* strides, const cuuint32_t* box, const cuuint32_t* elem_strides,
                 CUtensorMapSwizzle swizzle);
// Opt a kernel into `bytes` of dynamic shared memory once per (kernel, device).
int ensure_dynamic_smem(const void* kernel, int bytes);

int launch_linear_fp32(const float* x, const float* w, float* y, int M, int N, int K, cudaStream_t st);
int launch_rope_fp32(float* t, const float* cosv, const float* sinv, int B, int T, int H, int D,
                     long long cos_bstride, cudaStream_t st);
int launch_band_attn_fp32(const float* q, const float* k, const float* v, float* out, int B, int H, int D,
                          int Tq, int Tk, int q_off, int k_off, int window, float scale,
                          const long long* strides, cudaStream_t st);
int launch_qkv_rope_gemm(const void* x, const void* w_qkv, const QkvEpilogueArgs& ep, int M, int dtype_flags,
                         int* status, cudaStream_t st);
// y[M,512] = resid + out_scale * (a[M,512] * w[512,512]^T): the attention output projection with the layer
// scale and the residual add of the reference's transformer layer folded into the epilogue.
int launch_out_proj_gemm(const void* a, const void* w, void* y, const float* out_scale, const void* resid, int M,
                         int dtype_flags, int* status, cudaStream_t st);
// y[M,N] = resid + scale * act(a[M,K] * w[N,K]^T); in_dtype 0 BF16 / 1 FP16; out_dtype 0 BF16 / 1 FP16 / 2 FP32
// (type of y and resid); gelu 1 = exact GELU.  N a multiple of 256, K a multiple of 64.
int launch_linear_gemm(const void* a, const void* w, void* y, const float* scale, const void* resid, int M, int N,
                       int K, int in_dtype, int out_dtype, int gelu, int* status, cudaStream_t st);
// LayerNorm over 512 channels; x_dtype 0 BF16 / 1 FP16 / 2 FP32, y_dtype 0 BF16 / 1 FP16.
int launch_layernorm512(const void* x, int x_dtype, const float* weight, const float* bias, float eps, void* y,
                        int y_dtype, long long rows, cudaStream_t st);
// Residual vector quantisation (fm_rvq.cu): candidate selection + exact FP32 decision for one layer, FP16 copy of
// the residual, ordered FP32 decode.
int launch_rvq_select(const void* scores, int scores_fp16, const float* e_sq, const float* codebook, float* resid, void* resid16,
                      long long* codes, int* n_candidates, long long rows, int n_codes, float e_max, float tau_rel,
                      int* status, cudaStream_t st);
// Rows of a strided causal convolution with replicate padding, gathered from frame-major FP32 activations and split
// into FP16 hi + lo parts: [B * ceil(T / stride), kernel * C] (fm_downsample.cu).
int launch_conv_rows_split(const float* x, void* hi, void* lo, int B, int T, int C, int kernel, int stride,
                           cudaStream_t st);
int launch_wait_timeout_selftest(int* status, int limit_us, int* observed, cudaStream_t st);
// y[B, 2T, C] from x[B, T, C] by the depthwise transposed convolution of kernel 4, stride 2 (w [C, 4]), FP32.
int launch_upsample2_depthwise(const float* x, const float* w, float* y, int B, int T, int C, cudaStream_t st);
int launch_split_half(const float* x, void* hi, void* lo, long long n, cudaStream_t st);
// Record-based variant (no scores in memory): candidate records from launch_linear_gemm(out_dtype 3), per-frame
// margins in `tau` (written for the next layer by the decision kernel, for the first layer by launch_rvq_prepare).
int launch_rvq_select_rec(const void* records, const float* codebook, float* resid, void* resid16, long long* codes,
                          int* n_candidates, float* tau, long long rows, int n_codes, float e_max_next, float tau_rel,
                          int* status, cudaStream_t st);
int launch_rvq_prepare(const float* x, void* resid16, float* tau, long long rows, float e_max, float tau_rel,
                       cudaStream_t st);
int launch_rvq_to_half(const float* x, void* y, long long rows, cudaStream_t st);
int launch_rvq_decode(const long long* codes, const float* codebooks, float* out, long long rows, int n_layers,
                      int n_codes, int* bad_code, cudaStream_t st);
int launch_band_attn_prefill(const void* q, const void* k, const void* v, void* out, int B, int T, int window,
                             float scale, int value_is_fp16, int* status, cudaStream_t st);
// Queries [B, Tq, 512] against keys / values [B, Tk, 512], Tk >= Tq: the last Tq key rows are the queries' own
// frames, the Tk - Tq rows before them are older (cached) frames.
int launch_band_attn_chunk(const void* q, const void* k, const void* v, void* out, int B, int Tq, int Tk, int window,
                           float scale, int value_is_fp16, int* status, cudaStream_t st);
// KV ring <-> frame-major tensors for multi-frame cached calls (fm_ring.cu).
int launch_ring_linearize(const void* ring_k, const void* ring_v, const void* k_new, const void* v_new, void* k_lin,
                          void* v_lin, int S, int T, int delta, int past, int slots, cudaStream_t st);
int launch_ring_append(const void* k_new, const void* v_new, void* ring_k, void* ring_v, int S, int T, int past,
                       int slots, cudaStream_t st);
// Projection + RoPE + banded attention in one kernel for 128 < T <= 256 (fm_fused_clip.cu): q, k, v stay on chip.
int launch_attn_fused_clip(const void* x, const void* w_qkv, const float* cos, const float* sin, long long cos_bstride,
                           void* out, int B, int T, int window, float scale, int dtype_flags, int* status,
                           cudaStream_t st);
int launch_band_attn_clip(const void* q, const void* k, const void* v, void* out, int B, int T, int window,
                          float scale, int value_is_fp16, int* status, cudaStream_t st);
int launch_band_attn_long(const void* q, const void* k, const void* v, void* out, int B, int T, int window,
                          float scale, int value_is_fp16, int* status, cudaStream_t st);
int launch_ring_decode_attn(const void* q, const void* ring_k, const void* ring_v, float* out,
                            const int* stream_pos, int pos_base, int S, int ring_slots, float scale,
                            int value_is_fp16, int* status, cudaStream_t st);

}  // namespace fm
