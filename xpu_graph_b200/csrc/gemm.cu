// C-ABI front of the dense-layer kernels: argument validation and routing to the tensor-core
// (16-bit) or FFMA (fp32) implementation.
#include "common.cuh"

namespace xg {
struct GemmExtras;
int gemm_tc_entry(const void* A, const void* B, const void* bias, const void* residual, void* out, int64_t M, int64_t N,
                  int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr, int trans_b, int act, int dtype,
                  void* workspace, int64_t ws_bytes, cudaStream_t st, bool force_split = false,
                  const GemmExtras* extras = nullptr);
int64_t gemm_workspace_bytes(int64_t M, int64_t N, int64_t K);
int gemm_tc_static_entry(const void* A, const void* B, const void* bias, const void* residual, void* out, int64_t M,
                         int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr, int trans_b, int act,
                         int dtype, cudaStream_t st);
int64_t static_scratch_capacity();
int gemm_f32_entry(const void* A, const void* B, const void* bias, const void* residual, void* out, int64_t M, int64_t N,
                   int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr, int trans_b, int act, cudaStream_t st);
int gemm_swiglu_entry(const void* A, const void* Wg, const void* Wu, void* out, int64_t M, int64_t N, int64_t K,
                      int64_t lda, int64_t ldw, int64_t ldc, int dtype, cudaStream_t st);
int gemm_rope_entry(const void* A, const void* W, const void* cos, const void* sin, void* out, int64_t M, int64_t N, int64_t K,
                    int64_t lda, int64_t ldw, int64_t ldc, int64_t S, int64_t D, int dtype, cudaStream_t st);
int gemm_f32x3_entry(const void* A3, const void* W3, const void* bias, const void* residual, void* out, int64_t M,
                     int64_t N, int64_t Kp, int64_t ldc, int64_t ldr, int act, int out_planes, cudaStream_t st);
bool bgemm_single_launch_ok(const void* A, const void* B, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t lda,
                            int64_t ldb, int64_t sa, int64_t sb, int dtype);
int bgemm_tc_entry(const void* A, const void* B, const void* bias, const void* residual, void* out, int64_t batch, int64_t M,
                   int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr, int64_t sa, int64_t sb,
                   int64_t sbias, int64_t sr, int64_t sc, int trans_b, int act, int dtype, cudaStream_t st);
bool plan_ksplit(int64_t M, int64_t N, int64_t K, int dtype, int* S_out, int* tn_out);
int gemm_tc_ksplit_entry(const void* A, const void* W, const void* bias, const void* residual, void* out, int64_t M,
                         int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int act, int dtype, int S,
                         int tn, cudaStream_t st);
int gemm_group_entry(const void* const* A, const void* const* W, const void* const* bias, const void* const* residual,
                     void* const* out, int64_t count, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldc,
                     int64_t ldr, int trans_b, int act, int dtype, cudaStream_t st);
int gemm_simt16_entry(const void* A, const void* B, const void* bias, const void* residual, void* out, int64_t M, int64_t N,
                      int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr, int trans_b, int act, int dtype,
                      cudaStream_t st);
int gemm_f32_group_entry(const void* const* A, const void* const* W, const void* const* bias, const void* const* residual,
                         void* const* out, int64_t count, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldw,
                         int64_t ldc, int64_t ldr, int trans_b, int act, cudaStream_t st);
int read_tc_status(unsigned int* host_out, int reset);
int read_sdpa_status(unsigned int* host_out, int reset);
int read_ksplit_status(unsigned int* host_out, int reset);
int read_mlp_status(unsigned int* host_out, int reset);

namespace {
int validate_gemm(const char* name, const void* A, const void* B, const void* residual, void* out, int64_t M, int64_t N,
                  int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr, int trans_b, int act, int dtype) {
    if (!A || !B || !out) return fail(XG_ERR_INVALID_ARG, "%s: null A/B/out", name);
    if (M < 0 || N < 0 || K <= 0) return fail(XG_ERR_INVALID_ARG, "%s: bad extents M=%lld N=%lld K=%lld", name, (long long)M, (long long)N, (long long)K);
    if (dtype_size(dtype) == 0) return fail(XG_ERR_INVALID_ARG, "%s: bad dtype %d", name, dtype);
    if (act < XG_ACT_NONE || act > XG_ACT_SIGMOID) return fail(XG_ERR_INVALID_ARG, "%s: bad activation %d", name, act);
    if (lda < K || ldc < N || (residual && ldr < N)) return fail(XG_ERR_INVALID_ARG, "%s: leading dimension too small", name);
    if (ldb < (trans_b ? K : N)) return fail(XG_ERR_INVALID_ARG, "%s: ldb too small", name);
    return XG_OK;
}
}  // namespace
}  // namespace xg

extern "C" int xg_gemm_bias_act_ws(const void* A, const void* B, const void* bias, const void* residual, void* out,
                                   int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr,
                                   int trans_b, int act, int dtype, void* workspace, int64_t workspace_bytes,
                                   void* stream) {
    using namespace xg;
    int rc = validate_gemm("xg_gemm_bias_act", A, B, residual, out, M, N, K, lda, ldb, ldc, ldr, trans_b, act, dtype);
    if (rc != XG_OK) return rc;
    if (workspace_bytes < 0) return fail(XG_ERR_INVALID_ARG, "xg_gemm_bias_act_ws: negative workspace size");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (dtype == XG_F32) return gemm_f32_entry(A, B, bias, residual, out, M, N, K, lda, ldb, ldc, ldr, trans_b, act, st);
    // rows a tensor map cannot address (not multiples of 16 bytes from a 16-byte aligned base): the FMA kernel
    if (lda % 8 != 0 || ldb % 8 != 0 || (reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(B) & 15u))
        return gemm_simt16_entry(A, B, bias, residual, out, M, N, K, lda, ldb, ldc, ldr, trans_b, act, dtype, st);
    return gemm_tc_entry(A, B, bias, residual, out, M, N, K, lda, ldb, ldc, ldr, trans_b, act, dtype, workspace,
                         workspace_bytes, st);
}

extern "C" int xg_gemm_bias_act(const void* A, const void* B, const void* bias, const void* residual, void* out,
                                int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr,
                                int trans_b, int act, int dtype, void* stream) {
    return xg_gemm_bias_act_ws(A, B, bias, residual, out, M, N, K, lda, ldb, ldc, ldr, trans_b, act, dtype, nullptr, 0,
                               stream);
}

extern "C" int xg_gemm_bias_act_static(const void* A, const void* B, const void* bias, const void* residual, void* out,
                                       int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                                       int64_t ldr, int trans_b, int act, int dtype, void* stream) {
    using namespace xg;
    int rc = validate_gemm("xg_gemm_bias_act_static", A, B, residual, out, M, N, K, lda, ldb, ldc, ldr, trans_b, act, dtype);
    if (rc != XG_OK) return rc;
    if (dtype != XG_BF16 && dtype != XG_F16)
        return fail(XG_ERR_UNSUPPORTED, "xg_gemm_bias_act_static: 16-bit dtypes only (the fp32 kernel uses no scratch)");
    return gemm_tc_static_entry(A, B, bias, residual, out, M, N, K, lda, ldb, ldc, ldr, trans_b, act, dtype,
                                reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int xg_gemm_bias_act_cluster(const void* A, const void* W, const void* bias, const void* residual, void* out,
                                        int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr,
                                        int act, int dtype, int splits, int tile_n, void* stream) {
    using namespace xg;
    int rc = validate_gemm("xg_gemm_bias_act_cluster", A, W, residual, out, M, N, K, lda, ldw, ldc, ldr, 1, act, dtype);
    if (rc != XG_OK) return rc;
    if (dtype != XG_BF16 && dtype != XG_F16)
        return fail(XG_ERR_UNSUPPORTED, "xg_gemm_bias_act_cluster: 16-bit dtypes only");
    if ((reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(W) & 15u) || lda % 8 != 0 || ldw % 8 != 0)
        return fail(XG_ERR_UNSUPPORTED, "xg_gemm_bias_act_cluster: A/W must be 16-byte aligned with row strides multiple of 8 elements");
    if (M == 0 || N == 0) return XG_OK;
    if (M > (int64_t)256 * 0x7fff || N > (int64_t)64 * 0x7fffff || K > 0x7fffffff)
        return fail(XG_ERR_TOO_LARGE, "xg_gemm_bias_act_cluster: extent too large");
    return gemm_tc_ksplit_entry(A, W, bias, residual, out, M, N, K, lda, ldw, ldc, ldr, act, dtype, splits, tile_n,
                                reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int xg_gemm_cluster_plan(int64_t M, int64_t N, int64_t K, int dtype, int* splits, int* tile_n) {
    if (!splits || !tile_n || M <= 0 || N <= 0 || K <= 0 || (dtype != XG_BF16 && dtype != XG_F16)) return 0;
    return xg::plan_ksplit(M, N, K, dtype, splits, tile_n) ? 1 : 0;
}

extern "C" int64_t xg_gemm_static_scratch_bytes(void) { return xg::static_scratch_capacity(); }

extern "C" int64_t xg_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int dtype) {
    if (M <= 0 || N <= 0 || K <= 0 || (dtype != XG_BF16 && dtype != XG_F16)) return 0;
    return xg::gemm_workspace_bytes(M, N, K);
}

extern "C" int xg_bgemm_bias_act(const void* A, const void* B, const void* bias, const void* residual, void* out,
                                 int64_t batch, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                                 int64_t ldr, int64_t stride_a, int64_t stride_b, int64_t stride_bias, int64_t stride_r,
                                 int64_t stride_c, int trans_b, int act, int dtype, void* stream) {
    using namespace xg;
    if (batch < 0) return fail(XG_ERR_INVALID_ARG, "xg_bgemm_bias_act: negative batch");
    const int es = dtype_size(dtype);
    if (es == 0) return fail(XG_ERR_INVALID_ARG, "xg_bgemm_bias_act: bad dtype %d", dtype);
    if (batch == 0 || M * N == 0) return XG_OK;
    if (bgemm_single_launch_ok(A, B, batch, M, N, K, lda, ldb, stride_a, stride_b, dtype)) {
        int rc = validate_gemm("xg_bgemm_bias_act", A, B, residual, out, M, N, K, lda, ldb, ldc, ldr, trans_b, act, dtype);
        if (rc != XG_OK) return rc;
        return bgemm_tc_entry(A, B, bias, residual, out, batch, M, N, K, lda, ldb, ldc, ldr, stride_a, stride_b, stride_bias,
                              stride_r, stride_c, trans_b, act, dtype, reinterpret_cast<cudaStream_t>(stream));
    }
    for (int64_t b = 0; b < batch; ++b) {
        const char* Ab = reinterpret_cast<const char*>(A) + b * stride_a * es;
        const char* Bb = reinterpret_cast<const char*>(B) + b * stride_b * es;
        const char* biasb = bias ? reinterpret_cast<const char*>(bias) + b * stride_bias * es : nullptr;
        const char* rb = residual ? reinterpret_cast<const char*>(residual) + b * stride_r * es : nullptr;
        char* ob = reinterpret_cast<char*>(out) + b * stride_c * es;
        int rc = xg_gemm_bias_act(Ab, Bb, biasb, rb, ob, M, N, K, lda, ldb, ldc, ldr, trans_b, act, dtype, stream);
        if (rc != XG_OK) return rc;
    }
    return XG_OK;
}

extern "C" int xg_gemm_group_bias_act(const void* const* A, const void* const* W, const void* const* bias,
                                      const void* const* residual, void* const* out, int64_t count, int64_t M, int64_t N,
                                      int64_t K, int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int trans_b, int act,
                                      int dtype, void* stream) {
    using namespace xg;
    if (count < 0) return fail(XG_ERR_INVALID_ARG, "xg_gemm_group_bias_act: negative count");
    if (count == 0 || M == 0 || N == 0) return XG_OK;
    if (!A || !W || !out) return fail(XG_ERR_INVALID_ARG, "xg_gemm_group_bias_act: null pointer table");
    if (M < 0 || N < 0 || K <= 0) return fail(XG_ERR_INVALID_ARG, "xg_gemm_group_bias_act: bad extents");
    if (dtype != XG_BF16 && dtype != XG_F16 && dtype != XG_F32) return fail(XG_ERR_UNSUPPORTED, "xg_gemm_group_bias_act: unsupported dtype %d", dtype);
    if (act < XG_ACT_NONE || act > XG_ACT_SIGMOID) return fail(XG_ERR_INVALID_ARG, "xg_gemm_group_bias_act: bad activation %d", act);
    bool has_residual = false;
    for (int64_t e = 0; residual && e < count; ++e) has_residual = has_residual || residual[e] != nullptr;
    if (!has_residual) residual = nullptr;
    if (lda < K || ldc < N || ldw < (trans_b ? K : N) || (has_residual && ldr < N))
        return fail(XG_ERR_INVALID_ARG, "xg_gemm_group_bias_act: leading dimension too small");
    if (dtype == XG_F32)
        return gemm_f32_group_entry(A, W, bias, residual, out, count, M, N, K, lda, ldw, ldc, ldr, trans_b, act,
                                    reinterpret_cast<cudaStream_t>(stream));
    return gemm_group_entry(A, W, bias, residual, out, count, M, N, K, lda, ldw, ldc, ldr, trans_b, act, dtype,
                            reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int xg_gemm_swiglu(const void* A, const void* Wg, const void* Wu, void* out, int64_t M, int64_t N, int64_t K,
                              int64_t lda, int64_t ldw, int64_t ldc, int dtype, void* stream) {
    using namespace xg;
    if (!A || !Wg || !Wu || !out) return fail(XG_ERR_INVALID_ARG, "xg_gemm_swiglu: null pointer");
    if (M < 0 || N < 0 || K <= 0) return fail(XG_ERR_INVALID_ARG, "xg_gemm_swiglu: bad extents");
    if (dtype != XG_BF16 && dtype != XG_F16) return fail(XG_ERR_UNSUPPORTED, "xg_gemm_swiglu: 16-bit dtypes only");
    if (lda < K || ldw < K || ldc < N) return fail(XG_ERR_INVALID_ARG, "xg_gemm_swiglu: leading dimension too small");
    return gemm_swiglu_entry(A, Wg, Wu, out, M, N, K, lda, ldw, ldc, dtype, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int xg_gemm_rope(const void* A, const void* W, const void* cos, const void* sin, void* out, int64_t M, int64_t N,
                            int64_t K, int64_t lda, int64_t ldw, int64_t ldc, int64_t S, int64_t D, int dtype, void* stream) {
    using namespace xg;
    if (!A || !W || !cos || !sin || !out) return fail(XG_ERR_INVALID_ARG, "xg_gemm_rope: null pointer");
    if (M < 0 || N < 0 || K <= 0) return fail(XG_ERR_INVALID_ARG, "xg_gemm_rope: bad extents");
    if (dtype != XG_BF16 && dtype != XG_F16) return fail(XG_ERR_UNSUPPORTED, "xg_gemm_rope: 16-bit dtypes only");
    if (lda < K || ldw < K || ldc < N) return fail(XG_ERR_INVALID_ARG, "xg_gemm_rope: leading dimension too small");
    return gemm_rope_entry(A, W, cos, sin, out, M, N, K, lda, ldw, ldc, S, D, dtype, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int xg_gemm_f32x3(const void* A3, const void* W3, const void* bias, const void* residual, void* out, int64_t M,
                             int64_t N, int64_t K, int64_t ldc, int64_t ldr, int act, int out_planes, void* stream) {
    using namespace xg;
    if (!A3 || !W3 || !out) return fail(XG_ERR_INVALID_ARG, "xg_gemm_f32x3: null A3/W3/out");
    if (M < 0 || N < 0 || K <= 0) return fail(XG_ERR_INVALID_ARG, "xg_gemm_f32x3: bad extents");
    if (act < XG_ACT_NONE || act > XG_ACT_SIGMOID) return fail(XG_ERR_INVALID_ARG, "xg_gemm_f32x3: bad activation %d", act);
    if (!out_planes && (ldc < N || (residual && ldr < N))) return fail(XG_ERR_INVALID_ARG, "xg_gemm_f32x3: leading dimension too small");
    return gemm_f32x3_entry(A3, W3, bias, residual, out, M, N, xg_gemm_f32x3_padded_k(K), ldc, ldr, act, out_planes ? 1 : 0,
                            reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int xg_tc_status(unsigned int* status, int reset) {
    if (!status) return xg::fail(XG_ERR_INVALID_ARG, "xg_tc_status: null output");
    unsigned int a = 0, b = 0;
    int rc = xg::read_tc_status(&a, reset);
    if (rc != XG_OK) return rc;
    rc = xg::read_sdpa_status(&b, reset);
    if (rc != XG_OK) return rc;
    unsigned int c = 0;
    rc = xg::read_ksplit_status(&c, reset);
    if (rc != XG_OK) return rc;
    unsigned int d = 0;
    rc = xg::read_mlp_status(&d, reset);
    if (rc != XG_OK) return rc;
    *status = a | b | (c << 8) | (d << 16);
    return XG_OK;
}
