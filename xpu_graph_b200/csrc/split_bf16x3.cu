// fp32 -> three bf16 planes: x = x0 + x1 + x2 with x0 = bf16(x), x1 = bf16(x - x0), x2 = bf16(x - x0 - x1)
// (3 x 8 significand bits carry the 24 of fp32; the two subtractions are exact). The planes sit side by side in
// each output row, out[r][s * Kp + k], Kp = K rounded up to 64 and zero-filled, which is the operand layout of the
// fp32 GEMM that runs on the bf16 tensor cores (gemm_tc.cu, gemm_f32x3_entry).
//   transpose = 0: x is [rows, K] with row stride ld;  transpose = 1: x is [K, rows] (out row r = column r of x).
#include "common.cuh"

namespace xg {
namespace {

__device__ __forceinline__ void split3(float x, __nv_bfloat16& a, __nv_bfloat16& b, __nv_bfloat16& c) {
    a = __float2bfloat16_rn(x);
    const float r1 = x - __bfloat162float(a);
    b = __float2bfloat16_rn(r1);
    c = __float2bfloat16_rn(r1 - __bfloat162float(b));
}

template <bool TRANSPOSE>
__global__ void __launch_bounds__(256) split_bf16x3_kernel(const float* __restrict__ x, int64_t rows, int64_t K, int64_t ld,
                                                           int64_t Kp, __nv_bfloat16* __restrict__ out) {
    const int64_t groups = Kp / 8;  // 8 consecutive k per thread: one 16-byte store per plane
    const int64_t total = rows * groups;
    for (int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x; e < total; e += (int64_t)gridDim.x * 256) {
        int64_t r, g;
        if (TRANSPOSE) {  // neighbouring threads read neighbouring columns of x
            g = e / rows;
            r = e - g * rows;
        } else {
            r = e / groups;
            g = e - r * groups;
        }
        const int64_t k0 = g * 8;
        float v[8];
        if (!TRANSPOSE && k0 + 8 <= K && ((reinterpret_cast<uintptr_t>(x + r * ld + k0) & 15u) == 0)) {
            const float4 f0 = *reinterpret_cast<const float4*>(x + r * ld + k0);
            const float4 f1 = *reinterpret_cast<const float4*>(x + r * ld + k0 + 4);
            v[0] = f0.x; v[1] = f0.y; v[2] = f0.z; v[3] = f0.w;
            v[4] = f1.x; v[5] = f1.y; v[6] = f1.z; v[7] = f1.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int64_t k = k0 + i;
                v[i] = k < K ? (TRANSPOSE ? x[k * ld + r] : x[r * ld + k]) : 0.f;
            }
        }
        Vec16<__nv_bfloat16> p0, p1, p2;
#pragma unroll
        for (int i = 0; i < 8; ++i) split3(v[i], p0.v[i], p1.v[i], p2.v[i]);
        __nv_bfloat16* o = out + r * (3 * Kp) + k0;
        st16(o, p0);
        st16(o + Kp, p1);
        st16(o + 2 * Kp, p2);
    }
}

}  // namespace
}  // namespace xg

extern "C" int64_t xg_gemm_f32x3_padded_k(int64_t K) { return K <= 0 ? 0 : (K + 63) / 64 * 64; }

extern "C" int xg_split_bf16x3(const void* x, int64_t rows, int64_t K, int64_t ld, int transpose, void* out3, void* stream) {
    using namespace xg;
    if (rows < 0 || K < 0) return fail(XG_ERR_INVALID_ARG, "xg_split_bf16x3: negative extent");
    if (rows == 0 || K == 0) return XG_OK;
    if (!x || !out3) return fail(XG_ERR_INVALID_ARG, "xg_split_bf16x3: null pointer");
    if (ld < (transpose ? rows : K)) return fail(XG_ERR_INVALID_ARG, "xg_split_bf16x3: leading dimension too small");
    if (!aligned16(out3)) return fail(XG_ERR_UNSUPPORTED, "xg_split_bf16x3: the output must be 16-byte aligned");
    const int64_t Kp = xg_gemm_f32x3_padded_k(K);
    const int64_t work = (rows * (Kp / 8) + 255) / 256;
    const int64_t cap = 32LL * num_sms();
    const unsigned grid = (unsigned)(work < cap ? work : cap);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (transpose)
        split_bf16x3_kernel<true><<<grid, 256, 0, st>>>(reinterpret_cast<const float*>(x), rows, K, ld, Kp, reinterpret_cast<__nv_bfloat16*>(out3));
    else
        split_bf16x3_kernel<false><<<grid, 256, 0, st>>>(reinterpret_cast<const float*>(x), rows, K, ld, Kp, reinterpret_cast<__nv_bfloat16*>(out3));
    return check_launch("xg_split_bf16x3");
}
