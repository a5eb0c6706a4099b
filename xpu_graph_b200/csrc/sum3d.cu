// Batched reductions of 3-D tensors along one dim: out_t = sum(x_t, dim) for a list of contiguous [s0, s1, s2]
// tensors in one launch (grid.y = tensor). fp32 accumulation. HBM-bound: every input element is read once.
//   dim 1: one thread per output element (b, j), walking i -> loads coalesced across j;
//   dim 2: one warp per output element (b, i), lanes stride over j, shuffle reduction;
//   dim 0: one thread per output element (i, j), walking b.
#include "common.cuh"

namespace xg {
namespace {

constexpr int kMaxSumTensors = 64;

struct Sum3dParams {
    const void* in[kMaxSumTensors];
    void* out[kMaxSumTensors];
    int64_t s0[kMaxSumTensors];
    int32_t s1[kMaxSumTensors];
    int32_t s2[kMaxSumTensors];
    int32_t n;
    int32_t dim;
};

template <typename T>
__global__ void __launch_bounds__(256) sum3d_kernel(const __grid_constant__ Sum3dParams p) {
    const int t = blockIdx.y;
    const T* x = reinterpret_cast<const T*>(p.in[t]);
    T* o = reinterpret_cast<T*>(p.out[t]);
    const int64_t s0 = p.s0[t];
    const int s1 = p.s1[t], s2 = p.s2[t];
    if (p.dim == 1) {
        const int64_t total = s0 * s2;
        for (int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x; e < total; e += (int64_t)gridDim.x * 256) {
            const int64_t b = e / s2;
            const int j = (int)(e - b * s2);
            const T* src = x + b * s1 * (int64_t)s2 + j;
            float acc = 0.f;
            for (int i = 0; i < s1; ++i) acc += Cvt<T>::to_f(src[(int64_t)i * s2]);
            o[e] = Cvt<T>::from_f(acc);
        }
    } else if (p.dim == 2) {
        const int lane = threadIdx.x & 31;
        const int64_t rows = s0 * s1;
        for (int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); r < rows; r += (int64_t)gridDim.x * 8) {
            const T* src = x + r * s2;
            float acc = 0.f;
            for (int j = lane; j < s2; j += 32) acc += Cvt<T>::to_f(src[j]);
            acc = warp_sum(acc);
            if (lane == 0) o[r] = Cvt<T>::from_f(acc);
        }
    } else {
        const int64_t total = (int64_t)s1 * s2;
        for (int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x; e < total; e += (int64_t)gridDim.x * 256) {
            float acc = 0.f;
            for (int64_t b = 0; b < s0; ++b) acc += Cvt<T>::to_f(x[b * total + e]);
            o[e] = Cvt<T>::from_f(acc);
        }
    }
}

}  // namespace
}  // namespace xg

extern "C" int xg_sum3d(const void* const* inputs, void* const* outputs, const int64_t* shapes3, int64_t n, int dim,
                        int dtype, void* stream) {
    using namespace xg;
    if (n < 0) return fail(XG_ERR_INVALID_ARG, "xg_sum3d: negative count");
    if (dim < 0 || dim > 2) return fail(XG_ERR_INVALID_ARG, "xg_sum3d: dim must be 0, 1 or 2");
    if (dtype_size(dtype) == 0) return fail(XG_ERR_INVALID_ARG, "xg_sum3d: bad dtype %d", dtype);
    if (n == 0) return XG_OK;
    if (!inputs || !outputs || !shapes3) return fail(XG_ERR_INVALID_ARG, "xg_sum3d: null pointer");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    for (int64_t base = 0; base < n; base += kMaxSumTensors) {
        Sum3dParams p;
        p.n = 0;
        p.dim = dim;
        int64_t max_work = 0;
        for (int64_t k = base; k < n && p.n < kMaxSumTensors; ++k) {
            const int64_t s0 = shapes3[3 * k], s1 = shapes3[3 * k + 1], s2 = shapes3[3 * k + 2];
            if (s0 < 0 || s1 < 0 || s2 < 0 || s1 > 0x7fffffffLL || s2 > 0x7fffffffLL)
                return fail(XG_ERR_INVALID_ARG, "xg_sum3d: bad shape of tensor %lld", (long long)k);
            const int64_t out_elems = dim == 0 ? s1 * s2 : (dim == 1 ? s0 * s2 : s0 * s1);
            if (out_elems == 0) continue;
            if (!inputs[k] && s0 * s1 * s2 > 0) return fail(XG_ERR_INVALID_ARG, "xg_sum3d: null input %lld", (long long)k);
            if (!outputs[k]) return fail(XG_ERR_INVALID_ARG, "xg_sum3d: null output %lld", (long long)k);
            p.in[p.n] = inputs[k];
            p.out[p.n] = outputs[k];
            p.s0[p.n] = s0;
            p.s1[p.n] = (int32_t)s1;
            p.s2[p.n] = (int32_t)s2;
            const int64_t work = dim == 2 ? (out_elems + 7) / 8 : (out_elems + 255) / 256;
            if (work > max_work) max_work = work;
            p.n += 1;
        }
        if (p.n == 0) continue;
        const int64_t cap = 64LL * num_sms();
        const unsigned gx = (unsigned)(max_work < cap ? max_work : cap);
        dim3 grid(gx, (unsigned)p.n);
        switch (dtype) {
            case XG_F32: sum3d_kernel<float><<<grid, 256, 0, st>>>(p); break;
            case XG_BF16: sum3d_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p); break;
            default: sum3d_kernel<__half><<<grid, 256, 0, st>>>(p); break;
        }
        int rc = check_launch("xg_sum3d");
        if (rc != XG_OK) return rc;
    }
    return XG_OK;
}
