// Bandwidth-bound elementwise fusions: rotate-half RoPE and SwiGLU (silu(gate) * up).
// Both read each input element once with 16-byte loads and write the result once.
#include "common.cuh"

namespace xg {
namespace {

// ---------------------------------------------------------------------------------------
// RoPE. One thread produces the two 16-byte output vectors at column j and j + D/2 of a row,
// because both need the same pair of input vectors.
// ---------------------------------------------------------------------------------------
struct RopeParams {
    const void* x;
    const void* cos;
    const void* sin;
    void* y;
    int64_t B, H, S, D;
    int64_t sb, sh, ss;     // x strides (elements)
    int64_t yb, yh, ys;     // y strides (elements)
};

// grid.x covers (s, half-vector) of one (b, h) plane with 32-bit index math; grid.y strides over planes.
template <typename T>
__global__ void __launch_bounds__(256) rope_vec_kernel(const RopeParams p) {
    constexpr int EPV = Vec16<T>::N;
    const int hv_per_row = (int)(p.D / 2 / EPV);
    const uint32_t per_plane = (uint32_t)p.S * (uint32_t)hv_per_row;
    const uint32_t idx = blockIdx.x * 256u + threadIdx.x;
    if (idx >= per_plane) return;
    const uint32_t s = idx / (uint32_t)hv_per_row;
    const uint32_t hv = idx - s * (uint32_t)hv_per_row;
    const int64_t half = p.D / 2;
    const int64_t j = (int64_t)hv * EPV;
    const T* cr = reinterpret_cast<const T*>(p.cos) + (int64_t)s * p.D;
    const T* sr = reinterpret_cast<const T*>(p.sin) + (int64_t)s * p.D;
    const Vec16<T> c1 = ld16(cr + j), c2 = ld16(cr + j + half);
    const Vec16<T> s1 = ld16(sr + j), s2 = ld16(sr + j + half);
    const int64_t planes = p.B * p.H;
    for (int64_t bh = blockIdx.y; bh < planes; bh += gridDim.y) {
        const int64_t b = bh / p.H, h = bh - b * p.H;
        const T* xr = reinterpret_cast<const T*>(p.x) + b * p.sb + h * p.sh + (int64_t)s * p.ss;
        T* yr = reinterpret_cast<T*>(p.y) + b * p.yb + h * p.yh + (int64_t)s * p.ys;
        const Vec16<T> x1 = ld16_stream(xr + j), x2 = ld16_stream(xr + j + half);
        Vec16<T> o1, o2;
#pragma unroll
        for (int i = 0; i < EPV; ++i) {
            const float a = Cvt<T>::to_f(x1.v[i]), bb = Cvt<T>::to_f(x2.v[i]);
            o1.v[i] = Cvt<T>::from_f(a * Cvt<T>::to_f(c1.v[i]) - bb * Cvt<T>::to_f(s1.v[i]));
            o2.v[i] = Cvt<T>::from_f(bb * Cvt<T>::to_f(c2.v[i]) + a * Cvt<T>::to_f(s2.v[i]));
        }
        st16(yr + j, o1);
        st16(yr + j + half, o2);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) rope_scalar_kernel(const RopeParams p) {
    const int64_t half = p.D / 2;
    const int64_t total = p.B * p.H * p.S * half;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int64_t j = idx % half;
    const int64_t row = idx / half;
    const int64_t s = row % p.S;
    const int64_t bh = row / p.S;
    const int64_t h = bh % p.H;
    const int64_t b = bh / p.H;
    const T* xr = reinterpret_cast<const T*>(p.x) + b * p.sb + h * p.sh + s * p.ss;
    const T* cr = reinterpret_cast<const T*>(p.cos) + s * p.D;
    const T* sr = reinterpret_cast<const T*>(p.sin) + s * p.D;
    T* yr = reinterpret_cast<T*>(p.y) + b * p.yb + h * p.yh + s * p.ys;
    const float a = Cvt<T>::to_f(xr[j]), bb = Cvt<T>::to_f(xr[j + half]);
    yr[j] = Cvt<T>::from_f(a * Cvt<T>::to_f(cr[j]) - bb * Cvt<T>::to_f(sr[j]));
    yr[j + half] = Cvt<T>::from_f(bb * Cvt<T>::to_f(cr[j + half]) + a * Cvt<T>::to_f(sr[j + half]));
}

template <typename T>
int launch_rope(const RopeParams& p, cudaStream_t st) {
    constexpr int EPV = Vec16<T>::N;
    const int64_t half = p.D / 2;
    const bool vec_ok = (half % EPV == 0) && aligned16(p.x) && aligned16(p.cos) && aligned16(p.sin) && aligned16(p.y) &&
                        p.sb % EPV == 0 && p.sh % EPV == 0 && p.ss % EPV == 0 && p.yb % EPV == 0 && p.yh % EPV == 0 &&
                        p.ys % EPV == 0 && p.S * (half / EPV) < 0x7fffffffLL;
    if (vec_ok) {
        const int64_t per_plane = p.S * (half / EPV);
        const int64_t gx = (per_plane + 255) / 256;
        const int64_t planes = p.B * p.H;
        // enough CTAs to fill the GPU several times over, the rest of the planes are looped over
        int64_t gy = planes;
        const int64_t want = 32LL * num_sms();
        if (gx * gy > want) gy = (want + gx - 1) / gx;
        if (gy < 1) gy = 1;
        if (gy > 65535) gy = 65535;
        if (gy > planes) gy = planes;
        rope_vec_kernel<T><<<dim3((unsigned)gx, (unsigned)gy), 256, 0, st>>>(p);
    } else {
        const int64_t total = p.B * p.H * p.S * half;
        const int64_t grid = (total + 255) / 256;
        if (grid > 0x7fffffffLL) return fail(XG_ERR_TOO_LARGE, "xg_rope: tensor too large");
        rope_scalar_kernel<T><<<(unsigned)grid, 256, 0, st>>>(p);
    }
    return check_launch("xg_rope");
}

// ---------------------------------------------------------------------------------------
// SwiGLU
// ---------------------------------------------------------------------------------------
struct SwigluParams {
    const void* gate;
    const void* up;
    void* out;
    int64_t rows, cols, ldg, ldu, ldo;
};

// fp32 tensors use expf and a true division (the fp32 path must stay within 1e-5 relative of aten's
// silu); 16-bit tensors use silu(g) = h + h * tanh(h), h = g / 2, with the hardware tanh: one special-function
// operation per element instead of two, error about 2^-11 of the result (below a bf16 ulp, about one f16 ulp).
template <typename T>
__device__ __forceinline__ float silu_f(float g) {
    if (sizeof(T) == 4) return g / (1.0f + expf(-g));
    const float h = 0.5f * g;
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(h));
    return fmaf(h, t, h);
}

// One CTA owns ROWS consecutive rows; a thread walks the row's 16-byte vectors with stride 256 and handles the
// same column of all ROWS rows at once (2*ROWS loads in flight, no index division anywhere).
template <typename T, int ROWS>
__global__ void __launch_bounds__(256) swiglu_vec_kernel(const SwigluParams p) {
    constexpr int EPV = Vec16<T>::N;
    const int vec_per_row = (int)(p.cols / EPV);
    const int64_t r0 = (int64_t)blockIdx.x * ROWS;
    const T* gp = reinterpret_cast<const T*>(p.gate);
    const T* up = reinterpret_cast<const T*>(p.up);
    T* op = reinterpret_cast<T*>(p.out);
    for (int c = threadIdx.x; c < vec_per_row; c += 256) {
        Vec16<T> g[ROWS], u[ROWS];
#pragma unroll
        for (int k = 0; k < ROWS; ++k) {
            const int64_t r = r0 + k;
            if (r < p.rows) {
                g[k] = ld16_stream(gp + r * p.ldg + (int64_t)c * EPV);
                u[k] = ld16_stream(up + r * p.ldu + (int64_t)c * EPV);
            }
        }
#pragma unroll
        for (int k = 0; k < ROWS; ++k) {
            const int64_t r = r0 + k;
            if (r < p.rows) {
                Vec16<T> o;
#pragma unroll
                for (int i = 0; i < EPV; ++i)
                    o.v[i] = Cvt<T>::from_f(silu_f<T>(Cvt<T>::to_f(g[k].v[i])) * Cvt<T>::to_f(u[k].v[i]));
                st16(op + r * p.ldo + (int64_t)c * EPV, o);
            }
        }
    }
}

// Contiguous tensors (every row stride equals cols) are one long run of 16-byte vectors: a CTA takes 256 * U
// consecutive vectors and a thread U of them, 256 apart, so that a row length that is not a multiple of 256 vectors
// leaves no idle lanes at the end of every row.
template <typename T, int U>
__global__ void __launch_bounds__(256) swiglu_flat_kernel(const SwigluParams p, int64_t total_vec) {
    constexpr int EPV = Vec16<T>::N;
    const T* gp = reinterpret_cast<const T*>(p.gate);
    const T* up = reinterpret_cast<const T*>(p.up);
    T* op = reinterpret_cast<T*>(p.out);
    const int64_t v0 = (int64_t)blockIdx.x * (256 * U) + threadIdx.x;
    Vec16<T> g[U], u[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
        const int64_t v = v0 + k * 256;
        if (v < total_vec) {
            g[k] = ld16_stream(gp + v * EPV);
            u[k] = ld16_stream(up + v * EPV);
        }
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {
        const int64_t v = v0 + k * 256;
        if (v < total_vec) {
            Vec16<T> o;
#pragma unroll
            for (int i = 0; i < EPV; ++i)
                o.v[i] = Cvt<T>::from_f(silu_f<T>(Cvt<T>::to_f(g[k].v[i])) * Cvt<T>::to_f(u[k].v[i]));
            st16(op + v * EPV, o);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) swiglu_scalar_kernel(const SwigluParams p) {
    const int64_t total = p.rows * p.cols;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int64_t r = idx / p.cols, c = idx - r * p.cols;
    const float g = Cvt<T>::to_f(reinterpret_cast<const T*>(p.gate)[r * p.ldg + c]);
    const float u = Cvt<T>::to_f(reinterpret_cast<const T*>(p.up)[r * p.ldu + c]);
    reinterpret_cast<T*>(p.out)[r * p.ldo + c] = Cvt<T>::from_f(silu_f<T>(g) * u);
}

template <typename T>
int launch_swiglu(const SwigluParams& p, cudaStream_t st) {
    constexpr int EPV = Vec16<T>::N;
    constexpr int UNROLL = 4;
    const bool vec_ok = p.cols % EPV == 0 && p.ldg % EPV == 0 && p.ldu % EPV == 0 && p.ldo % EPV == 0 &&
                        aligned16(p.gate) && aligned16(p.up) && aligned16(p.out);
    const bool flat = p.ldg == p.cols && p.ldu == p.cols && p.ldo == p.cols;
    if (vec_ok && flat) {
        const int64_t total_vec = p.rows * (p.cols / EPV);
        const int64_t grid = (total_vec + 256 * UNROLL - 1) / (256 * UNROLL);
        if (grid > 0x7fffffffLL) return fail(XG_ERR_TOO_LARGE, "xg_swiglu: tensor too large");
        if (grid > 0) swiglu_flat_kernel<T, UNROLL><<<(unsigned)grid, 256, 0, st>>>(p, total_vec);
    } else if (vec_ok && p.cols / EPV < 0x7fffffffLL) {
        const int64_t grid = (p.rows + UNROLL - 1) / UNROLL;
        if (grid > 0x7fffffffLL) return fail(XG_ERR_TOO_LARGE, "xg_swiglu: tensor too large");
        swiglu_vec_kernel<T, UNROLL><<<(unsigned)grid, 256, 0, st>>>(p);
    } else {
        const int64_t grid = (p.rows * p.cols + 255) / 256;
        if (grid > 0x7fffffffLL) return fail(XG_ERR_TOO_LARGE, "xg_swiglu: tensor too large");
        swiglu_scalar_kernel<T><<<(unsigned)grid, 256, 0, st>>>(p);
    }
    return check_launch("xg_swiglu");
}

}  // namespace
}  // namespace xg

extern "C" int xg_rope(const void* x, const void* cos, const void* sin, void* y, int64_t B, int64_t H, int64_t S,
                       int64_t D, int64_t x_stride_b, int64_t x_stride_h, int64_t x_stride_s, int64_t y_stride_b,
                       int64_t y_stride_h, int64_t y_stride_s, int dtype, void* stream) {
    using namespace xg;
    if (!x || !cos || !sin || !y) return fail(XG_ERR_INVALID_ARG, "xg_rope: null pointer");
    if (B < 0 || H < 0 || S < 0 || D <= 0 || (D & 1)) return fail(XG_ERR_INVALID_ARG, "xg_rope: bad extents (D must be even)");
    if (dtype_size(dtype) == 0) return fail(XG_ERR_INVALID_ARG, "xg_rope: bad dtype %d", dtype);
    if (B * H * S == 0) return XG_OK;
    RopeParams p{x, cos, sin, y, B, H, S, D, x_stride_b, x_stride_h, x_stride_s, y_stride_b, y_stride_h, y_stride_s};
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    switch (dtype) {
        case XG_F32: return launch_rope<float>(p, st);
        case XG_BF16: return launch_rope<__nv_bfloat16>(p, st);
        default: return launch_rope<__half>(p, st);
    }
}

extern "C" int xg_swiglu(const void* gate, const void* up, void* out, int64_t rows, int64_t cols, int64_t ld_gate,
                         int64_t ld_up, int64_t ld_out, int dtype, void* stream) {
    using namespace xg;
    if (!gate || !up || !out) return fail(XG_ERR_INVALID_ARG, "xg_swiglu: null pointer");
    if (rows < 0 || cols < 0) return fail(XG_ERR_INVALID_ARG, "xg_swiglu: negative extent");
    if (ld_gate < cols || ld_up < cols || ld_out < cols) return fail(XG_ERR_INVALID_ARG, "xg_swiglu: row stride smaller than cols");
    if (dtype_size(dtype) == 0) return fail(XG_ERR_INVALID_ARG, "xg_swiglu: bad dtype %d", dtype);
    if (rows * cols == 0) return XG_OK;
    SwigluParams p{gate, up, out, rows, cols, ld_gate, ld_up, ld_out};
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    switch (dtype) {
        case XG_F32: return launch_swiglu<float>(p, st);
        case XG_BF16: return launch_swiglu<__nv_bfloat16>(p, st);
        default: return launch_swiglu<__half>(p, st);
    }
}
