/*
 * xg_sm100 — C ABI of the sm_100a kernel library behind xpu_graph's `cuda_sm100` target.
 *
 * Conventions (all entry points):
 *   - plain pointers and sizes; the caller owns every buffer (device memory unless the
 *     parameter is documented as a HOST array);
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*) of the caller's current
 *     device; nothing synchronises the device, nothing allocates device memory;
 *   - return value: XG_OK (0) or a negative XG_ERR_* code; the library never aborts or throws;
 *     xg_last_error() returns a thread-local, human-readable message for the last failure;
 *   - dtype codes: XG_F32 / XG_BF16 / XG_F16; element strides ("ld", "stride") are in ELEMENTS
 *     unless the name ends in _bytes.
 *
 * Each declaration cites the reference interface it stands in for (paths are relative to the
 * xpu_graph source tree, src/xpu_graph/...).
 */
#ifndef XG_SM100_H_
#define XG_SM100_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XG_OK 0
#define XG_ERR_INVALID_ARG (-1)   /* null pointer, negative extent, bad enum */
#define XG_ERR_UNSUPPORTED (-2)   /* shape / dtype / alignment this build has no kernel for */
#define XG_ERR_LAUNCH (-3)        /* cudaGetLastError() after the launch was not cudaSuccess */
#define XG_ERR_DEVICE (-4)        /* wrong architecture or no device */
#define XG_ERR_TOO_LARGE (-5)     /* size beyond a documented fixed maximum */

#define XG_F32 0
#define XG_BF16 1
#define XG_F16 2

#define XG_ACT_NONE 0
#define XG_ACT_GELU 1 /* erf form, aten.gelu(approximate='none') */
#define XG_ACT_RELU 2
#define XG_ACT_SILU 3
#define XG_ACT_SIGMOID 4

/* ---- library identity ------------------------------------------------------------------ */

/* ABI version of this header (major*1000 + minor). */
int xg_version(void);
/* 1 if device `device` is compute capability 10.x (the only architecture the kernels are built for). */
int xg_device_arch_ok(int device);
/* Message of the last failing call on this thread ("" if none). */
const char* xg_last_error(void);

/*
 * Status word of the tensor-core kernels on the current device: 0 = healthy; non-zero = a bounded
 * wait inside a kernel expired (bit 0 producer, bit 1 MMA issuer, bit 2 epilogue, bits 4-6 the same
 * roles of the attention kernel, bits 8-10 of the cluster dense kernel, bits 16-18 of the chained-layer kernel) and that
 * launch's output is invalid. This is the one entry point
 * that synchronises (it copies the word back); reset != 0 clears it. No reference counterpart.
 */
int xg_tc_status(unsigned int* status, int reset);

/* ---- normalisation --------------------------------------------------------------------- */

/*
 * RMSNorm with optional fused residual add.
 *   s = residual ? round_to_dtype(x + residual) : x
 *   y = to_dtype( (float(s) * rsqrt(mean(float(s)^2) + eps)) * float(weight) )
 *   if sum_out: sum_out = s          (the "store output before norm" second result)
 * Replaces: passes/patterns/utils/default_replacements.py:19-25 (DefaultRMSNorm) as called by
 * passes/patterns/structure/custom_rmsnorm.py:21-29; residual form: targets/npu/triton_kernel/
 * fused_add_rmsnorm.py:10-36 and targets/mlu/fuse_add_norm.py:21-83 (store_output_before_norm).
 * x, residual, y, sum_out: [rows, hidden], last dim contiguous, row strides in elements
 * (y and sum_out are written with row stride `hidden`). weight: [hidden] of dtype w_dtype
 * (XG_F32 or the same as dtype).
 */
int xg_rmsnorm(const void* x, const void* residual, const void* weight, void* y, void* sum_out,
               int64_t rows, int64_t hidden, int64_t x_row_stride, int64_t res_row_stride,
               float eps, int dtype, int w_dtype, void* stream);

/*
 * LayerNorm with optional fused residual add; weight is required (as in
 * passes/patterns/structure/custom_layernorm.py:25), bias may be null (layer_norm(..., bias=None), the configuration of
 * the reference's own residual-add test, tests/mlu/test_fuse_addlayernorm.py:39-43).
 *   s = residual ? round_to_dtype(x + residual) : x
 *   y = to_dtype( (float(s) - mean) * rsqrt(var + eps) * float(weight) + float(bias) )
 * Replaces: passes/patterns/utils/default_replacements.py:28-36 (DefaultLayerNorm) as called by
 * passes/patterns/structure/custom_layernorm.py:21-29; residual form targets/mlu/fuse_add_norm.py:21-83.
 */
int xg_layernorm(const void* x, const void* residual, const void* weight, const void* bias, void* y,
                 void* sum_out, int64_t rows, int64_t hidden, int64_t x_row_stride,
                 int64_t res_row_stride, float eps, int dtype, int w_dtype, void* stream);

/* ---- elementwise fusions --------------------------------------------------------------- */

/*
 * Rotate-half rotary embedding: y = x*cos + cat(-x[..., D/2:], x[..., :D/2])*sin.
 * x, y: [B, H, S, D], each addressed by element strides (D contiguous), so a [B, S, H, D] buffer
 * viewed as [B, H, S, D] is read and written in place of a transpose copy; cos/sin: [S, D]
 * contiguous, same dtype as x. The reference has no RoPE op; this replaces the 2x slice + neg + cat +
 * 2x mul + add chain that the graph carries (semantics of the aten ops).
 */
int xg_rope(const void* x, const void* cos, const void* sin, void* y, int64_t B, int64_t H, int64_t S,
            int64_t D, int64_t x_stride_b, int64_t x_stride_h, int64_t x_stride_s, int64_t y_stride_b,
            int64_t y_stride_h, int64_t y_stride_s, int dtype, void* stream);

/*
 * SwiGLU: out = silu(gate) * up, row-major [rows, cols] with separate row strides (a packed
 * [rows, 2*cols] tensor is passed as gate = base, up = base + cols, both ld = 2*cols).
 * Replaces: targets/npu/triton_kernel/fused_silu_mul.py:10-60 (fused_silu_mul).
 */
int xg_swiglu(const void* gate, const void* up, void* out, int64_t rows, int64_t cols, int64_t ld_gate,
              int64_t ld_up, int64_t ld_out, int dtype, void* stream);

/* ---- dense layers ---------------------------------------------------------------------- */

/*
 * out[M,N] = act( A[M,K] @ W + bias + residual ),  W = B[K,N] (trans_b = 0) or B[N,K]^T (trans_b = 1).
 * bias: nullable [N]; residual: nullable [M,N] with row stride ldr (the "2-D bias" / beta = 1 form);
 * act: XG_ACT_*. dtype XG_BF16 / XG_F16: tensor-core path (tcgen05, fp32 accumulate) when A and B are
 * 16-byte aligned with row strides that are multiples of 8 elements; other 16-bit operands run on the
 * FMA kernel (elements converted on the way in and out, fp32 accumulate) - correct for any extents, meant
 * for small layers. dtype XG_F32: true fp32 FMA path (no TF32).
 * Replaces: targets/mlu/structure_replacements/dense_layer_modules.py:9-57 (DenseLayerModule →
 * torch_mlu_ops.matmul) as called by passes/patterns/structure/custom_denselayer.py:80-88.
 */
int xg_gemm_bias_act(const void* A, const void* B, const void* bias, const void* residual, void* out,
                     int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                     int64_t ldr, int trans_b, int act, int dtype, void* stream);

/*
 * Same as xg_gemm_bias_act with caller-provided scratch memory. For small M (few output tiles) the
 * 16-bit kernel splits K over several CTAs per tile: each writes its fp32 partial sums to `workspace`
 * ([splits][M][N] floats) and a second pass reduces them in a fixed order (deterministic) and applies
 * bias / residual / activation. xg_gemm_workspace_bytes returns the size this shape would like (0 when
 * splitting does not pay); a smaller or null workspace only lowers the split factor. The workspace
 * must be 16-byte aligned device memory; its contents before and after the call are unspecified.
 * Reference counterpart: the same torch_mlu_ops.matmul call site as xg_gemm_bias_act.
 */
int xg_gemm_bias_act_ws(const void* A, const void* B, const void* bias, const void* residual, void* out,
                        int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                        int64_t ldr, int trans_b, int act, int dtype, void* workspace,
                        int64_t workspace_bytes, void* stream);
int64_t xg_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int dtype);

/*
 * The same dense layer (16-bit dtypes, W given as [N,K]) on the thread-block-cluster kernel with the caller's
 * choice of decomposition: every 256 x `tile_n` output tile is computed by a cluster of `splits` CTA pairs, each
 * pair taking a share of K, and the partial tiles are added through distributed shared memory in split order
 * (deterministic; no scratch memory, no second launch). splits in 1..4; tile_n a multiple of 32 in 64..256 with
 * tile_n / 32 >= splits; K must span at least `splits` 64-wide blocks. xg_gemm_bias_act picks this kernel (and
 * these two numbers) by itself for problems with few output tiles; xg_gemm_cluster_plan reports that choice
 * (returns 1 and fills splits / tile_n, or 0 when it would run another kernel). For autotuners and tests.
 * Reference counterpart: the same torch_mlu_ops.matmul call site as xg_gemm_bias_act
 * (targets/mlu/structure_replacements/dense_layer_modules.py:9-57).
 */
int xg_gemm_bias_act_cluster(const void* A, const void* W, const void* bias, const void* residual, void* out,
                             int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr,
                             int act, int dtype, int splits, int tile_n, void* stream);
int xg_gemm_cluster_plan(int64_t M, int64_t N, int64_t K, int dtype, int* splits, int* tile_n);

/*
 * Split-K dense layer for hosts that cannot allocate device memory. Some embedders of this library own
 * no allocator they may call at this point: a plugin running inside another framework's stream-ordered
 * memory pool, a runtime whose memory budget was fixed at start-up, or a real-time serving loop in which a
 * cudaMalloc (an implicit device synchronisation) is not acceptable. For them the fp32 partial sums go to a
 * 32 MiB array that is part of the library image (xg_gemm_static_scratch_bytes() returns the size; every GPU
 * that loads the library holds it until the process exits) instead of a caller workspace. Inputs and outputs
 * are still the caller's. Same arithmetic as xg_gemm_bias_act_ws with a 2-way or wider split.
 *   - 16-bit dtypes only; XG_ERR_TOO_LARGE when 2*M*N*4 bytes exceed the array (M*N > 4 Mi elements),
 *     XG_ERR_UNSUPPORTED when K fits a single 64-wide k-block.
 *   - The first call on each device resolves the array's device address (cudaGetSymbolAddress, a short
 *     host-side set-up step); make that first call before starting any stream capture.
 *   - No cudaMalloc / cudaFree / allocating library call is made, on the first call or later.
 *   - All calls share the one array and it keeps whatever the previous call left there; every partial
 *     sum that is read has been written earlier in the same call, so nothing needs clearing. Two calls
 *     whose kernels overlap on the GPU (different streams, or several host threads) race on the array:
 *     serialise them.
 * This entry point has no counterpart in the reference.
 */
int xg_gemm_bias_act_static(const void* A, const void* B, const void* bias, const void* residual, void* out,
                            int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                            int64_t ldr, int trans_b, int act, int dtype, void* stream);
int64_t xg_gemm_static_scratch_bytes(void);

/*
 * fp32 dense layer on the bf16 tensor cores. Each fp32 operand is first cut into three bf16 planes
 * (x = x0 + x1 + x2, 3 x 8 significand bits) laid side by side per row: xg_split_bf16x3 writes
 * out3[r][s * Kp + k], Kp = xg_gemm_f32x3_padded_k(K) (K rounded up to 64, zero-filled), from x [rows, K]
 * (transpose = 0, row stride ld) or from x [K, rows] (transpose = 1). xg_gemm_f32x3 then computes
 * act(A @ W^T + bias + residual) in fp32 from A3 [M, 3*Kp] and W3 [N, 3*Kp] (the six plane products of
 * weight >= 2^-16, fp32 accumulation): results agree with an fp32 FMA GEMM to about 1e-6 relative. bias [N] and
 * residual [M, ldr] are fp32. out_planes = 0: out is fp32 [M, ldc]. out_planes = 1: out receives the result already
 * cut into planes, [M, 3 * xg_gemm_f32x3_padded_k(N)] bf16 with the padding columns zero, i.e. the A3 of a following
 * layer (no residual in this form). A weight's planes can be kept across calls.
 * Same reference interface as xg_gemm_bias_act (dense_layer_modules.py:9-57) for fp32 tensors; chaining layers
 * through plane outputs stands where the reference fuses serial matmuls (targets/mlu/fuse_densetower.py:272-316).
 */
int64_t xg_gemm_f32x3_padded_k(int64_t K);
int xg_split_bf16x3(const void* x, int64_t rows, int64_t K, int64_t ld, int transpose, void* out3, void* stream);
int xg_gemm_f32x3(const void* A3, const void* W3, const void* bias, const void* residual, void* out, int64_t M,
                  int64_t N, int64_t K, int64_t ldc, int64_t ldr, int act, int out_planes, void* stream);

/*
 * Batched form: out[b] = act( A[b] @ W[b] + bias[b] + residual[b] ), batch strides in elements
 * (0 broadcasts). 16-bit problems with positive, 16-byte aligned operand strides run as ONE launch over
 * (entry, tile) work units; fp32 and broadcast operands run entry by entry.
 * Replaces: dense_layer_modules.py:71-120 (BatchDenseLayerModule) as called by
 * passes/patterns/structure/custom_denselayer.py:111-117; also the stacked-bmm form of
 * targets/mlu/combo_matmul.py:53-87 (FusedCombineBmm.forward_bmm).
 */
int xg_bgemm_bias_act(const void* A, const void* B, const void* bias, const void* residual, void* out,
                      int64_t batch, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                      int64_t ldc, int64_t ldr, int64_t stride_a, int64_t stride_b,
                      int64_t stride_bias, int64_t stride_r, int64_t stride_c, int trans_b, int act,
                      int dtype, void* stream);

/*
 * Two or three chained dense layers in one kernel: out = act2( act1( x @ W1^T + b1 ) @ W2^T + b2 ) (and a third layer
 * on top for xg_mlp3_bias_act), x [M, K1], W1 [N1, K1], W2 [N2, N1], W3 [N3, N2] as nn.Linear stores them, or - for
 * every layer l whose bit (1 << l) is set in weights_kn - as [K, N] (the operand of torch.matmul(x, W), the form of the
 * reference's own test, tests/mlu/test_fuse_densetower.py:18-35; such a weight's N must be a multiple of 8);
 * out [M, N_last]; row strides in elements; biases nullable. The hidden activations stay on chip: each is rounded to
 * the 16-bit dtype (as the unfused graph rounds it when it stores the tensor) and handed to the next product through
 * shared memory. 16-bit dtypes only; xg_mlp2_supported / xg_mlp3_supported say whether a shape fits (K1 % 8 == 0, every
 * width <= 256, hidden widths >= 16 and multiples of 8); x and the weights 16-byte aligned with row strides that are
 * multiples of 8 elements.
 * Replaces: FusedDenseTower2Replacement.forward -> fuse_serial_mm_2dot and FusedDenseTower3Replacement.forward ->
 * fuse_serial_mm_3dot (targets/mlu/fuse_densetower.py:14-49, 80-131, matched by FusedDenseTower2 / 3 :272-316; kernels
 * triton_kernel/fused_serial_mm_2dot.py:142, fused_serial_mm_3dot.py:271), whose condition is likewise that the weights
 * fit on chip (:66-77).
 */
int xg_mlp2_supported(int64_t M, int64_t K1, int64_t N1, int64_t N2, int dtype);
int xg_mlp3_supported(int64_t M, int64_t K1, int64_t N1, int64_t N2, int64_t N3, int dtype);
int xg_mlp2_bias_act(const void* x, const void* w1, const void* b1, const void* w2, const void* b2, void* out, int64_t M,
                     int64_t K1, int64_t N1, int64_t N2, int64_t lda, int64_t ldw1, int64_t ldw2, int64_t ldc, int act1,
                     int act2, int weights_kn, int dtype, void* stream);
int xg_mlp3_bias_act(const void* x, const void* w1, const void* b1, const void* w2, const void* b2, const void* w3,
                     const void* b3, void* out, int64_t M, int64_t K1, int64_t N1, int64_t N2, int64_t N3, int64_t lda,
                     int64_t ldw1, int64_t ldw2, int64_t ldw3, int64_t ldc, int act1, int act2, int act3, int weights_kn,
                     int dtype, void* stream);

/*
 * Small dense tower: 1..3 chained layers y = act_l(y @ W_l + b_l) whose widths (dims[0..layers]: the input width, then
 * each layer's) are all <= 128 and whose weights together hold at most 24576 elements, as ONE kernel: every weight
 * stays in shared memory for the whole launch and the hidden activations never leave the SM. fp32 / bf16 / f16, any
 * row length or alignment (plain loads, FMA arithmetic with fp32 accumulation; fp32 towers are exact fp32); hidden
 * activations are rounded to the tensors' dtype once per layer. w, bias (nullable table, nullable entries), ldw and
 * act are host arrays with one entry per layer; bit l of weights_kn says that W_l is stored [K, N] instead of [N, K].
 * xg_mlp_small_supported answers whether a tower qualifies (no device call).
 * Replaces: the serial-matmul kernels of targets/mlu/fuse_densetower.py:272-316 at the sizes of their own condition
 * "the weights fit on chip" (:66-77; tests/mlu/test_fuse_densetower.py:36-53 runs 16 rows of 20 -> 32 -> 16 -> 1 in fp16).
 */
int xg_mlp_small_supported(const int64_t* dims, int layers, int dtype);
int xg_mlp_small_bias_act(const void* x, const void* const* w, const void* const* bias, void* out, int64_t M,
                          const int64_t* dims, int layers, int64_t lda, const int64_t* ldw, int64_t ldc, const int* act,
                          int weights_kn, int dtype, void* stream);

/*
 * Grouped form: out[e] = act( A[e] @ W[e] + bias[e] + residual[e] ) for `count` problems of one shape [M, N, K] whose
 * operands lie wherever the caller has them: A, W, bias, residual (nullable tables, nullable entries; bias[e] a row of N,
 * residual[e] an [M, N] matrix with row stride ldr) and out are host arrays of `count` device pointers, so nothing is
 * stacked or copied. 16-bit dtypes: one launch per 12 entries walks (entry, tile) work units with each entry's own
 * tensor maps; every A[e] / W[e] 16-byte aligned, lda / ldw multiples of 8 elements. fp32: one launch per 24 entries of
 * the FMA kernels (true fp32, any alignment), the entry being the grid's third dimension.
 * Replaces: the grouped-GEMM form of targets/mlu/combo_matmul.py:87-113 (FusedCombineBmm.forward_groupgemm ->
 * torch.ops.torch_mlu.grouped_gemm), emitted by FusedCombineMatMul (:116-232).
 */
int xg_gemm_group_bias_act(const void* const* A, const void* const* W, const void* const* bias,
                           const void* const* residual, void* const* out, int64_t count, int64_t M, int64_t N, int64_t K,
                           int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int trans_b, int act, int dtype, void* stream);

/*
 * Dual GEMM with SwiGLU epilogue: out = silu(A @ Wg^T) * (A @ Wu^T); Wg, Wu: [N, K] (Linear layout).
 * Replaces the mul(silu(mm), mm) sub-graph; elementwise part as targets/npu/fuse_silu_mul.py:21-69.
 */
int xg_gemm_swiglu(const void* A, const void* Wg, const void* Wu, void* out, int64_t M, int64_t N,
                   int64_t K, int64_t lda, int64_t ldw, int64_t ldc, int dtype, void* stream);

/*
 * Projection with the rotary embedding in the epilogue: out[r, :] = rope(round(A[r, :] @ W^T)) per head, where row
 * r is token (r / S, r % S), heads are consecutive blocks of D output columns, and cos/sin are [S, D] tables of
 * the output dtype (rotate-half form, as xg_rope). W: [N, K] Linear layout, N % D == 0, D in {64, 128}. The
 * projection result is rounded to the tensor dtype before the rotation, as the un-fused graph does.
 * Replaces: the dense layer (structure/custom_denselayer.py:80-88) followed by the RoPE chain of xg_rope.
 */
int xg_gemm_rope(const void* A, const void* W, const void* cos, const void* sin, void* out, int64_t M, int64_t N,
                 int64_t K, int64_t lda, int64_t ldw, int64_t ldc, int64_t S, int64_t D, int dtype, void* stream);

/* ---- attention ------------------------------------------------------------------------- */

/*
 * out = softmax(q @ k^T * scale + mask) @ v, per (batch, head); online softmax, fp32 accumulate.
 * q: [B,H,Sq,D], k,v: [B,H,Skv,D], out: [B,H,Sq,D]; each addressed by element strides for
 * (batch, head, seq) with D contiguous. mask: nullable additive mask of the same dtype,
 * addressed by element strides for (batch, head, q, kv) — 0 strides broadcast. causal != 0 applies
 * the lower-triangular mask aligned to the top-left corner (query i sees keys j <= i), as
 * aten.scaled_dot_product_attention(is_causal=True) does.
 * Replaces: aten.scaled_dot_product_attention as emitted by
 * passes/patterns/common/fuse_scaled_dot_product_attention.py:163-238 (FusedSDPA).
 */
int xg_sdpa_fwd(const void* q, const void* k, const void* v, const void* mask, void* out, int64_t B,
                int64_t H, int64_t Sq, int64_t Skv, int64_t D, const int64_t* q_strides3,
                const int64_t* k_strides3, const int64_t* v_strides3, const int64_t* o_strides3,
                const int64_t* mask_strides4, float scale, int causal, int dtype, void* stream);

/* ---- copy fusions (bit-exact) ---------------------------------------------------------- */

/*
 * Segmented 2-D copy: for every segment k and row r < rows,
 *   dst_k[r*dst_ld_k + 0..len_k) = zero_row(r) ? 0 : src_k[r*src_ld_k + 0..len_k)
 * where src_k = (char*)src_ptrs[k], dst_k = (char*)dst_ptrs[k]; all lengths and strides in BYTES.
 * zero_row(r) = row_mask && (row_mask[r] != 0) == (mask_zero_when != 0); row_mask: nullable
 * device bytes [rows]. src_ptrs/dst_ptrs/src_ld_bytes/dst_ld_bytes/len_bytes: HOST arrays of nseg.
 * This one entry point carries: slice+cat of one source (targets/mlu/structure_replacements/
 * __init__.py:50-63, FuseSliceCatSameInputModule), equal-length multi-slice to [num, rows, len]
 * (:21-47, FuseSliceModule), multi-output split (:66-144, FuseSliceCatSameInputModule_v2),
 * where-masked slice+cat (targets/mlu/triton_kernel/fused_slice_where_cat.py:12-73), and plain
 * cat / stack of several sources along the last dim.
 */
int xg_seg_copy(const void* const* src_ptrs, void* const* dst_ptrs, const int64_t* src_ld_bytes,
                const int64_t* dst_ld_bytes, const int64_t* len_bytes, int64_t nseg, int64_t rows,
                const uint8_t* row_mask, int mask_zero_when, void* stream);

/*
 * Multi-table row gather (embedding lookups fused with the where-mask and the stack/cat):
 *   out[r*out_ld + f*D + j] = zero_row(r) ? 0 : tables[f][idx(r,f)*D + j],   j < D
 * tables: HOST array of F device pointers to [table_rows[f], D] contiguous tables;
 * idx(r,f) = idx[r*idx_row_stride + f*idx_col_stride] (int64, device); an index outside
 * [0, table_rows[f]) writes zeros for that row. elem_size in {2,4,8}; out_ld in elements.
 * Replaces: F fused aten.embedding lookups + where + stack; nearest reference anchors are
 * targets/mlu/repeat_to_expand.py:25-56 and torch_mlu.emb_concat
 * (targets/mlu/structure_replacements/__init__.py:136).
 */
int xg_gather_rows(const void* const* tables, const int64_t* table_rows, int64_t F, const int64_t* idx,
                   int64_t idx_row_stride, int64_t idx_col_stride, const uint8_t* row_mask,
                   int mask_zero_when, void* out, int64_t rows, int64_t D, int64_t out_ld,
                   int elem_size, void* stream);

/*
 * Batched sum over one dim of n contiguous 3-D tensors in one launch: outputs[k] = sum(inputs[k], dim),
 * shapes3 = HOST array [n][3] of (s0, s1, s2); dim 0 -> [s1, s2], dim 1 -> [s0, s2], dim 2 -> [s0, s1]
 * (contiguous, same dtype, fp32 accumulation). inputs/outputs: HOST arrays of device pointers.
 * Replaces: targets/mlu/triton_kernel/fused_sum_3d.py:131-205 (fused_sum_3d_input) as called by
 * targets/mlu/structure_replacements/__init__.py:147-165 (ComboSumModule) for
 * passes/patterns/structure/fuse_combosum.py:82-98 (ComboSum3dInp).
 */
int xg_sum3d(const void* const* inputs, void* const* outputs, const int64_t* shapes3, int64_t n, int dim,
             int dtype, void* stream);

/*
 * Row reductions written side by side: out[b, k*C + c] = sum over r in [r0_k, r1_k) of
 * a_k[b, r, c] * (b_ptrs ? b_k[b, r, c] : 1) for k = 0..n-1. a_k / b_k are contiguous [*, R_k, C] tensors addressed
 * as base + b * batch_stride + r * C + c (a batch stride of 0 broadcasts one slab over the batch); row_ranges2 =
 * HOST array [n][2] of (r0, r1); a_ptrs / b_ptrs / strides: HOST arrays. out: [B, out_ld] with out_ld >= n*C.
 * fp32 accumulation. When all segments read one tensor from the same first row every input row is read once.
 * Replaces: targets/mlu/triton_kernel/fused_slice_sum_cat.py (fuse_slice_sum_cat) as called by
 * targets/mlu/fuse_sum_cat.py:76-115 (SliceSumCatOperation, pattern FusedCatSum :242-252), and
 * targets/mlu/triton_kernel/fused_mul_sum_cat.py (fused_mul_sum_cat_2inp) as called by
 * targets/mlu/fuse_mul_sum_cat.py:16-50 (FusedMulSumCatReplacement, pattern FusedMulSumCat :97-123).
 */
int xg_rowsum_cat(const void* const* a_ptrs, const void* const* b_ptrs, const int64_t* a_batch_strides,
                  const int64_t* b_batch_strides, const int64_t* row_ranges2, int64_t n, int64_t B, int64_t C,
                  void* out, int64_t out_ld, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* XG_SM100_H_ */
