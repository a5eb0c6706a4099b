// True-fp32 dense layer (no TF32): out = act(A @ W + bias + residual) with FFMA accumulation.
// Shared-memory tiled SIMT kernel; used for the fp32 graphs whose tolerance (1e-5 relative) rules out
// tensor-core TF32, and - with 16-bit elements converted on the way in and out, fp32 in between - for the 16-bit
// shapes whose rows no tensor map can address (row lengths or base addresses that are not multiples of 16 bytes). W is [K, N] (trans_b = 0) or [N, K] (trans_b = 1); both tiles are stored k-major
// in shared memory so the inner product reads float4 vectors without bank conflicts.
#include "common.cuh"

namespace xg {
namespace {

struct GemmF32Params {  // element type: the kernel's template parameter
    const void* A;
    const void* B;
    const void* bias;
    const void* residual;
    void* out;
    int64_t M, N, K, lda, ldb, ldc, ldr;
    int trans_b;
    int act;
};

__device__ __forceinline__ float act_f32(float v, int act) {
    switch (act) {
        case XG_ACT_GELU: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
        case XG_ACT_RELU: return v > 0.f ? v : 0.f;
        case XG_ACT_SILU: return v / (1.0f + expf(-v));
        case XG_ACT_SIGMOID: return 1.0f / (1.0f + expf(-v));
        default: return v;
    }
}

// 256 threads; thread (ty, tx) owns a TM x TN micro-tile; BM = 16*TM, BN = 16*TN.
template <typename T, int TM, int TN, int BK>
__device__ __forceinline__ void gemm_f32_tile(const GemmF32Params& p) {
    constexpr int BM = 16 * TM, BN = 16 * TN;
    const T* __restrict__ gA = reinterpret_cast<const T*>(p.A);
    const T* __restrict__ gB = reinterpret_cast<const T*>(p.B);
    const T* gbias = reinterpret_cast<const T*>(p.bias);
    const T* gres = reinterpret_cast<const T*>(p.residual);
    T* gout = reinterpret_cast<T*>(p.out);
    __shared__ __align__(16) float As[2][BK][BM + 4];
    __shared__ __align__(16) float Bs[2][BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    constexpr int A_ELEMS = BM * BK / 256;
    constexpr int B_ELEMS = BN * BK / 256;
    float a_reg[A_ELEMS], b_reg[B_ELEMS];

    auto load_global = [&](int64_t k0) {
#pragma unroll
        for (int e = 0; e < A_ELEMS; ++e) {
            const int idx = tid + e * 256;  // k fastest: consecutive threads read consecutive k of one row
            const int kk = idx % BK, mm = idx / BK;
            const int64_t gm = m0 + mm, gk = k0 + kk;
            a_reg[e] = (gm < p.M && gk < p.K) ? Cvt<T>::to_f(gA[gm * p.lda + gk]) : 0.f;
        }
#pragma unroll
        for (int e = 0; e < B_ELEMS; ++e) {
            const int idx = tid + e * 256;
            if (p.trans_b) {  // W[N, K]: k fastest
                const int kk = idx % BK, nn = idx / BK;
                const int64_t gn = n0 + nn, gk = k0 + kk;
                b_reg[e] = (gn < p.N && gk < p.K) ? Cvt<T>::to_f(gB[gn * p.ldb + gk]) : 0.f;
            } else {  // W[K, N]: n fastest
                const int nn = idx % BN, kk = idx / BN;
                const int64_t gn = n0 + nn, gk = k0 + kk;
                b_reg[e] = (gn < p.N && gk < p.K) ? Cvt<T>::to_f(gB[gk * p.ldb + gn]) : 0.f;
            }
        }
    };
    auto store_shared = [&](int buf) {
#pragma unroll
        for (int e = 0; e < A_ELEMS; ++e) {
            const int idx = tid + e * 256;
            As[buf][idx % BK][idx / BK] = a_reg[e];
        }
#pragma unroll
        for (int e = 0; e < B_ELEMS; ++e) {
            const int idx = tid + e * 256;
            if (p.trans_b) Bs[buf][idx % BK][idx / BK] = b_reg[e];
            else Bs[buf][idx / BN][idx % BN] = b_reg[e];
        }
    };

    const int64_t nk = (p.K + BK - 1) / BK;
    load_global(0);
    store_shared(0);
    __syncthreads();
    for (int64_t kt = 0; kt < nk; ++kt) {
        const int buf = (int)(kt & 1);
        if (kt + 1 < nk) load_global((kt + 1) * BK);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; i += 4) {
                const float4 t = *reinterpret_cast<const float4*>(&As[buf][kk][ty * TM + i]);
                a[i] = t.x; a[i + 1] = t.y; a[i + 2] = t.z; a[i + 3] = t.w;
            }
#pragma unroll
            for (int j = 0; j < TN; j += 4) {
                const float4 t = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * TN + j]);
                b[j] = t.x; b[j + 1] = t.y; b[j + 2] = t.z; b[j + 3] = t.w;
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (kt + 1 < nk) {
            store_shared(buf ^ 1);
            __syncthreads();
        }
    }

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int64_t gm = m0 + ty * TM + i;
        if (gm >= p.M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int64_t gn = n0 + tx * TN + j;
            if (gn >= p.N) continue;
            float v = acc[i][j];
            if (gbias) v += Cvt<T>::to_f(gbias[gn]);
            if (gres) v += Cvt<T>::to_f(gres[gm * p.ldr + gn]);
            gout[gm * p.ldc + gn] = Cvt<T>::from_f(act_f32(v, p.act));
        }
    }
}

template <typename T, int TM, int TN, int BK>
__global__ void __launch_bounds__(256) gemm_f32_kernel(const GemmF32Params p) {
    gemm_f32_tile<T, TM, TN, BK>(p);
}

// Grouped form: blockIdx.z picks the entry; its five pointers come from a table in the kernel's parameter space, the
// extents, strides and activation are shared by the group.
constexpr int kF32GroupMax = 24;  // 24 x 5 pointers = 960 bytes of parameters
struct GemmF32Group {
    const void* A[kF32GroupMax];
    const void* B[kF32GroupMax];
    const void* bias[kF32GroupMax];
    const void* residual[kF32GroupMax];
    void* out[kF32GroupMax];
};
__device__ __forceinline__ GemmF32Params entry_params(const GemmF32Params& p, const GemmF32Group& g) {
    GemmF32Params pe = p;
    const int e = blockIdx.z;
    pe.A = g.A[e];
    pe.B = g.B[e];
    pe.bias = g.bias[e];
    pe.residual = g.residual[e];
    pe.out = g.out[e];
    return pe;
}

template <typename T, int TM, int TN, int BK>
__global__ void __launch_bounds__(256) gemm_f32_group_kernel(const GemmF32Params p, const __grid_constant__ GemmF32Group g) {
    const GemmF32Params pe = entry_params(p, g);
    gemm_f32_tile<T, TM, TN, BK>(pe);
}

// Small problems (fewer 64 x 64 tiles than SMs) are latency-bound in the kernel above: every 16-wide k-tile costs a
// round trip to L2. This variant gives each CTA a small output tile and the whole K-panel of both operands, 256 k at
// a time, fetched with one burst of 16-byte asynchronous copies, so a k-chunk costs one round trip; the inner
// product reads both panels as float4 along k (A rows are shared by the 16 threads of a row group, the B rows of the
// 8 threads of a wavefront fall into distinct bank groups with the 260-float row pitch). W must be [N, K].
// 128 threads as 8 (m) x 16 (n); thread (ty, tx) owns a TM x TN micro-tile; BM = 8 TM, BN = 16 TN.
constexpr int kPanelK = 256;
constexpr int kPanelPitch = kPanelK + 4;  // floats; rows stay 16-byte aligned

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(bytes) : "memory");
}

template <int TM, int TN>
__device__ __forceinline__ void gemm_f32_panel_tile(const GemmF32Params& p) {
    constexpr int BM = 8 * TM, BN = 16 * TN;
    extern __shared__ __align__(16) float panel[];
    float* As = panel;                      // [BM][kPanelPitch]
    float* Bs = panel + BM * kPanelPitch;   // [BN][kPanelPitch]
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int64_t k0 = 0; k0 < p.K; k0 += kPanelK) {
        const int kc = (int)((p.K - k0) < kPanelK ? (p.K - k0) : kPanelK);  // multiple of 4 (host-checked)
        const int vec_per_row = kc / 4;
        if (k0 > 0) __syncthreads();  // the previous chunk has been consumed
        for (int idx = tid; idx < BM * vec_per_row; idx += 128) {
            const int r = idx / vec_per_row, v = idx - r * vec_per_row;
            const int64_t gm = m0 + r;
            cp_async16(As + r * kPanelPitch + 4 * v, reinterpret_cast<const float*>(p.A) + (gm < p.M ? gm : 0) * p.lda + k0 + 4 * v, gm < p.M);
        }
        for (int idx = tid; idx < BN * vec_per_row; idx += 128) {
            const int r = idx / vec_per_row, v = idx - r * vec_per_row;
            const int64_t gn = n0 + r;
            cp_async16(Bs + r * kPanelPitch + 4 * v, reinterpret_cast<const float*>(p.B) + (gn < p.N ? gn : 0) * p.ldb + k0 + 4 * v, gn < p.N);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        // unrolled: with two or three warps per scheduler the shared-memory loads of several k-steps have to be in
        // flight together (one k-step per iteration ran at 7.9 cycles per issued instruction)
#pragma unroll 4
        for (int k = 0; k < kc; k += 4) {
            float4 a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = *reinterpret_cast<const float4*>(As + (ty * TM + i) * kPanelPitch + k);
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = *reinterpret_cast<const float4*>(Bs + (tx * TN + j) * kPanelPitch + k);
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    float c = acc[i][j];
                    c = fmaf(a[i].x, b[j].x, c);
                    c = fmaf(a[i].y, b[j].y, c);
                    c = fmaf(a[i].z, b[j].z, c);
                    c = fmaf(a[i].w, b[j].w, c);
                    acc[i][j] = c;
                }
        }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int64_t gm = m0 + ty * TM + i;
        if (gm >= p.M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int64_t gn = n0 + tx * TN + j;
            if (gn >= p.N) continue;
            float v = acc[i][j];
            if (p.bias) v += reinterpret_cast<const float*>(p.bias)[gn];
            if (p.residual) v += reinterpret_cast<const float*>(p.residual)[gm * p.ldr + gn];
            reinterpret_cast<float*>(p.out)[gm * p.ldc + gn] = act_f32(v, p.act);
        }
    }
}

template <int TM, int TN>
__global__ void __launch_bounds__(128) gemm_f32_panel_kernel(const GemmF32Params p) {
    gemm_f32_panel_tile<TM, TN>(p);
}

template <int TM, int TN>
__global__ void __launch_bounds__(128) gemm_f32_panel_group_kernel(const GemmF32Params p, const __grid_constant__ GemmF32Group g) {
    const GemmF32Params pe = entry_params(p, g);
    gemm_f32_panel_tile<TM, TN>(pe);
}

template <int TM, int TN>
int launch_panel_group(const GemmF32Params& p, const GemmF32Group& g, int count, cudaStream_t st) {
    constexpr int BM = 8 * TM, BN = 16 * TN;
    constexpr int smem = (BM + BN) * kPanelPitch * (int)sizeof(float);
    auto kern = gemm_f32_panel_group_kernel<TM, TN>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(XG_ERR_LAUNCH, "xg_gemm_group_bias_act(f32): cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    dim3 grid((unsigned)((p.N + BN - 1) / BN), (unsigned)((p.M + BM - 1) / BM), (unsigned)count);
    kern<<<grid, 128, smem, st>>>(p, g);
    return check_launch("xg_gemm_group_bias_act(f32)");
}

template <int TM, int TN>
int launch_panel(const GemmF32Params& p, cudaStream_t st) {
    constexpr int BM = 8 * TM, BN = 16 * TN;
    constexpr int smem = (BM + BN) * kPanelPitch * (int)sizeof(float);
    auto kern = gemm_f32_panel_kernel<TM, TN>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(XG_ERR_LAUNCH, "xg_gemm_bias_act(f32): cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    dim3 grid((unsigned)((p.N + BN - 1) / BN), (unsigned)((p.M + BM - 1) / BM));
    kern<<<grid, 128, smem, st>>>(p);
    return check_launch("xg_gemm_bias_act(f32)");
}

}  // namespace

int gemm_f32_entry(const void* A, const void* B, const void* bias, const void* residual, void* out, int64_t M, int64_t N,
                   int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr, int trans_b, int act, cudaStream_t st) {
    if (M * N == 0) return XG_OK;
    GemmF32Params p{A, B, bias, residual, out, M, N, K, lda, ldb, ldc, ldr, trans_b, act};
    const int64_t tiles64 = ((M + 63) / 64) * ((N + 63) / 64);
    const bool panel_ok = trans_b && K % 4 == 0 && lda % 4 == 0 && ldb % 4 == 0 && aligned16(A) && aligned16(B) &&
                          (M + 15) / 16 <= 65535;
    if (panel_ok && tiles64 < num_sms()) {  // latency-bound sizes: small tiles, whole K-panels per round trip
        const int64_t tiles_32x64 = ((M + 31) / 32) * ((N + 63) / 64);
        if (tiles_32x64 * 3 >= 2LL * num_sms()) return launch_panel<4, 4>(p, st);
        return launch_panel<2, 2>(p, st);
    }
    const int64_t big_tiles = ((M + 127) / 128) * ((N + 127) / 128);
    if (big_tiles >= 2LL * num_sms()) {
        dim3 grid((unsigned)((N + 127) / 128), (unsigned)((M + 127) / 128));
        if ((M + 127) / 128 > 65535) return fail(XG_ERR_TOO_LARGE, "xg_gemm_bias_act(f32): M too large");
        gemm_f32_kernel<float, 8, 8, 16><<<grid, 256, 0, st>>>(p);
    } else {
        dim3 grid((unsigned)((N + 63) / 64), (unsigned)((M + 63) / 64));
        if ((M + 63) / 64 > 65535) return fail(XG_ERR_TOO_LARGE, "xg_gemm_bias_act(f32): M too large");
        gemm_f32_kernel<float, 4, 4, 16><<<grid, 256, 0, st>>>(p);
    }
    return check_launch("xg_gemm_bias_act(f32)");
}

// 16-bit operands the tensor-core kernels cannot address (rows or base addresses that are not multiples of 16 bytes):
// the same tiled FMA kernel, elements converted on the way in and out, fp32 accumulation.
int gemm_simt16_entry(const void* A, const void* B, const void* bias, const void* residual, void* out, int64_t M, int64_t N,
                      int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr, int trans_b, int act, int dtype,
                      cudaStream_t st) {
    if (M * N == 0) return XG_OK;
    GemmF32Params p{A, B, bias, residual, out, M, N, K, lda, ldb, ldc, ldr, trans_b, act};
    const bool big = ((M + 127) / 128) * ((N + 127) / 128) >= 2LL * num_sms();
    const int64_t bm = big ? 128 : 64;
    if ((M + bm - 1) / bm > 65535) return fail(XG_ERR_TOO_LARGE, "xg_gemm_bias_act: M too large for the unaligned 16-bit path");
    dim3 grid((unsigned)((N + bm - 1) / bm), (unsigned)((M + bm - 1) / bm));
    if (dtype == XG_BF16) {
        if (big) gemm_f32_kernel<__nv_bfloat16, 8, 8, 16><<<grid, 256, 0, st>>>(p);
        else gemm_f32_kernel<__nv_bfloat16, 4, 4, 16><<<grid, 256, 0, st>>>(p);
    } else {
        if (big) gemm_f32_kernel<__half, 8, 8, 16><<<grid, 256, 0, st>>>(p);
        else gemm_f32_kernel<__half, 4, 4, 16><<<grid, 256, 0, st>>>(p);
    }
    return check_launch("xg_gemm_bias_act (16-bit, FMA path)");
}

// out[e] = act(A[e] @ W[e] + bias[e] + residual[e]) for `count` fp32 problems of one shape; the operands stay where
// they are (a pointer per entry). One launch per 24 entries; the kernel is chosen as for a single problem with `count`
// times the tiles.
int gemm_f32_group_entry(const void* const* A, const void* const* W, const void* const* bias, const void* const* residual,
                         void* const* out, int64_t count, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldw,
                         int64_t ldc, int64_t ldr, int trans_b, int act, cudaStream_t st) {
    if (M * N == 0) return XG_OK;
    if ((M + 15) / 16 > 65535) return fail(XG_ERR_TOO_LARGE, "xg_gemm_group_bias_act(f32): M too large");
    for (int64_t first = 0; first < count; first += kF32GroupMax) {
        const int n = (int)((count - first) < kF32GroupMax ? (count - first) : kF32GroupMax);
        GemmF32Group g;
        bool aligned = true;
        for (int e = 0; e < kF32GroupMax; ++e) {
            const int64_t i = first + (e < n ? e : 0);  // unused slots repeat the first entry and are never read
            if (!A[i] || !W[i] || !out[i])
                return fail(XG_ERR_INVALID_ARG, "xg_gemm_group_bias_act: null pointer in entry %lld", (long long)i);
            g.A[e] = A[i];
            g.B[e] = W[i];
            g.bias[e] = bias ? bias[i] : nullptr;
            g.residual[e] = residual ? residual[i] : nullptr;
            g.out[e] = out[i];
            aligned = aligned && aligned16(A[i]) && aligned16(W[i]);
        }
        GemmF32Params p{nullptr, nullptr, nullptr, nullptr, nullptr, M, N, K, lda, ldw, ldc, ldr, trans_b, act};
        const int64_t tiles64 = ((M + 63) / 64) * ((N + 63) / 64) * n;
        const bool panel_ok = trans_b && K % 4 == 0 && lda % 4 == 0 && ldw % 4 == 0 && aligned;
        int rc;
        if (panel_ok && tiles64 < num_sms()) {
            const int64_t tiles_32x64 = ((M + 31) / 32) * ((N + 63) / 64) * n;
            rc = tiles_32x64 * 3 >= 2LL * num_sms() ? launch_panel_group<4, 4>(p, g, n, st) : launch_panel_group<2, 2>(p, g, n, st);
        } else if (((M + 127) / 128) * ((N + 127) / 128) * n >= 2LL * num_sms()) {
            dim3 grid((unsigned)((N + 127) / 128), (unsigned)((M + 127) / 128), (unsigned)n);
            gemm_f32_group_kernel<float, 8, 8, 16><<<grid, 256, 0, st>>>(p, g);
            rc = check_launch("xg_gemm_group_bias_act(f32)");
        } else {
            dim3 grid((unsigned)((N + 63) / 64), (unsigned)((M + 63) / 64), (unsigned)n);
            gemm_f32_group_kernel<float, 4, 4, 16><<<grid, 256, 0, st>>>(p, g);
            rc = check_launch("xg_gemm_group_bias_act(f32)");
        }
        if (rc != XG_OK) return rc;
    }
    return XG_OK;
}

}  // namespace xg
