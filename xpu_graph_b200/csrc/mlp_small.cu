// Small dense tower: up to three chained layers y = act(y @ W + b) whose widths are all <= 128, as ONE kernel with every
// weight resident in shared memory for the whole launch and the hidden activations never leaving the SM. This is the
// regime of the reference's serial-matmul fusion (targets/mlu/fuse_densetower.py:66-77: "the weights fit on chip";
// its own test runs 16 rows through 20 -> 32 -> 16 -> 1 in fp16, tests/mlu/test_fuse_densetower.py:36-53): widths far
// below a tensor-core tile, rows no tensor map can address, a problem that is launch-bound as separate layers.
//
// 256 threads per CTA; a CTA converts the weights to fp32 in shared memory once ([K][N], n fastest, for either storage
// order), then walks blocks of 32 rows: the block's input rows go to shared memory as fp32, and for each layer thread
// (n, g) owns column n of the layer for the rows of group g (256 / pow2(N) groups share out the 32 rows), reading the
// weight column once per k and the activations as broadcast float4 along k. fp32 accumulation; hidden activations are
// rounded to the tensors' dtype once, after the activation, as the unfused graph's tensors are; fp32 towers are exact
// FMA arithmetic (no TF32).
#include "common.cuh"

namespace xg {
namespace {

constexpr int MS_THREADS = 256;
constexpr int MS_ROWS = 32;            // rows per block of work
constexpr int MS_MAX_DIM = 128;        // widest layer (and widest input)
constexpr int MS_BATCH = 4;            // loads in flight per thread while filling shared memory
constexpr int MS_MAX_WEIGHT_FLOATS = 24576;  // 96 KiB of fp32 weights in shared memory

struct MlpSmallParams {
    const void* x;
    const void* w[3];
    const void* bias[3];
    void* out;
    int64_t M, lda, ldc, ldw[3];
    int dims[4];   // K0, N1, N2, N3
    int act[3];
    int layers;
    int w_kn;      // bit l: weight l is stored [K, N] (else [N, K])
};

__device__ __forceinline__ float ms_act(float v, int act) {
    switch (act) {
        case XG_ACT_GELU: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
        case XG_ACT_RELU: return v > 0.f ? v : 0.f;
        case XG_ACT_SILU: return v / (1.0f + expf(-v));
        case XG_ACT_SIGMOID: return 1.0f / (1.0f + expf(-v));
        default: return v;
    }
}

__host__ __device__ __forceinline__ int ms_pad4(int k) { return (k + 3) & ~3; }
__host__ __device__ __forceinline__ int ms_pow2(int n) {
    int p = 1;
    while (p < n) p <<= 1;
    return p;
}

// One layer for one block of rows: thread (n, g) owns column n for rows [g * RPT, g * RPT + RPT). RPT is a template
// parameter (1, 2, 4, 8 or 16 = pow2(N) / 8) so that no predicated-off row costs an issue slot; not inlined, so that a
// launch executes one compact copy per row count (a CTA that serves 16 rows is bound by instruction fetch).
template <typename T, int RPT>
__device__ __noinline__ void ms_layer(const float* __restrict__ in, float* __restrict__ nxt, const float* __restrict__ wcol,
                                      float bias, int N, int Kp, int pitch, int r_lo, int n, int act, T* out_rows, int64_t ldc,
                                      int rows) {
    float acc[RPT];
#pragma unroll
    for (int j = 0; j < RPT; ++j) acc[j] = bias;
    const float* a_row = in + r_lo * pitch;
    for (int k = 0; k < Kp; k += 4) {
        const float w0 = wcol[k * N], w1 = wcol[(k + 1) * N], w2 = wcol[(k + 2) * N], w3 = wcol[(k + 3) * N];
#pragma unroll
        for (int j = 0; j < RPT; ++j) {
            const float4 a = *reinterpret_cast<const float4*>(a_row + j * pitch + k);
            float c = acc[j];
            c = fmaf(a.x, w0, c);
            c = fmaf(a.y, w1, c);
            c = fmaf(a.z, w2, c);
            c = fmaf(a.w, w3, c);
            acc[j] = c;
        }
    }
#pragma unroll
    for (int j = 0; j < RPT; ++j) {
        const int r = r_lo + j;
        const T v = Cvt<T>::from_f(ms_act(acc[j], act));
        if (out_rows != nullptr) {
            if (r < rows) out_rows[(int64_t)r * ldc + n] = v;
        } else {
            nxt[r * pitch + n] = Cvt<T>::to_f(v);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(MS_THREADS) mlp_small_kernel(const MlpSmallParams p) {
    extern __shared__ __align__(16) float ms_smem[];
    // [weights of layer 0 | 1 | 2: Kp x N each, rows k >= K zero][biases][activation buffer A][activation buffer B]
    float* w_s[3] = {ms_smem, ms_smem, ms_smem};
    float* b_s[3] = {ms_smem, ms_smem, ms_smem};
    float* cur = ms_smem;
    int max_dim = p.dims[0];
    for (int l = 0; l < p.layers; ++l) {
        w_s[l] = cur;
        cur += ms_pad4(p.dims[l]) * p.dims[l + 1];
        if (p.dims[l + 1] > max_dim) max_dim = p.dims[l + 1];
    }
    for (int l = 0; l < p.layers; ++l) {
        b_s[l] = cur;
        cur += ms_pad4(p.dims[l + 1]);
    }
    const int pitch = ms_pad4(max_dim) + 4;  // floats per activation row; keeps rows 16-byte aligned
    float* act_a = cur;
    float* act_b = cur + MS_ROWS * pitch;
    const int tid = threadIdx.x;

    // Filling shared memory. A CTA that serves 16 rows spends its life waiting on memory, so the loads of ALL layers'
    // weights and biases (MS_BATCH elements per thread and layer) go out before any of them is used: one trip to memory
    // per pass over the three layers instead of one per layer and batch.
    {
        int totals[3], max_total = 0;
#pragma unroll
        for (int l = 0; l < 3; ++l) {
            totals[l] = l < p.layers ? ms_pad4(p.dims[l]) * p.dims[l + 1] : 0;
            if (totals[l] > max_total) max_total = totals[l];
        }
        for (int base = tid; base < max_total; base += MS_BATCH * MS_THREADS) {
            float v[3][MS_BATCH];
            int dst[3][MS_BATCH];
#pragma unroll
            for (int l = 0; l < 3; ++l) {
                const bool used = l < p.layers;  // unused layers: extents that divide, nothing loaded or stored
                const int K = used ? p.dims[l] : 4, N = used ? p.dims[l + 1] : 1, Kp = ms_pad4(K);
                const T* __restrict__ w = reinterpret_cast<const T*>(p.w[l]);
                const bool kn = (p.w_kn >> l) & 1;
                const int64_t ldw = p.ldw[l];
#pragma unroll
                for (int u = 0; u < MS_BATCH; ++u) {
                    const int idx = base + u * MS_THREADS;
                    // consecutive threads read consecutive elements of the stored rows
                    int k, n;
                    if (kn) { k = idx / N; n = idx - k * N; }
                    else { n = idx / Kp; k = idx - n * Kp; }
                    const bool in = idx < totals[l];
                    dst[l][u] = in ? k * N + n : -1;
                    v[l][u] = (in && k < K) ? Cvt<T>::to_f(kn ? w[(int64_t)k * ldw + n] : w[(int64_t)n * ldw + k]) : 0.f;
                }
            }
            float bv[3];
#pragma unroll
            for (int l = 0; l < 3; ++l) {  // the biases ride in the first pass (widths <= 128 < MS_THREADS)
                const T* b = reinterpret_cast<const T*>(p.bias[l]);
                bv[l] = (base == tid && l < p.layers && b != nullptr && tid < p.dims[l + 1]) ? Cvt<T>::to_f(b[tid]) : 0.f;
            }
#pragma unroll
            for (int l = 0; l < 3; ++l) {
#pragma unroll
                for (int u = 0; u < MS_BATCH; ++u)
                    if (dst[l][u] >= 0) w_s[l][dst[l][u]] = v[l][u];
                if (base == tid && l < p.layers && tid < p.dims[l + 1]) b_s[l][tid] = bv[l];
            }
        }
    }

    const T* __restrict__ x = reinterpret_cast<const T*>(p.x);
    T* out = reinterpret_cast<T*>(p.out);
    const int64_t blocks = (p.M + MS_ROWS - 1) / MS_ROWS;
    for (int64_t blk = blockIdx.x; blk < blocks; blk += gridDim.x) {
        const int64_t row0 = blk * MS_ROWS;
        const int rows = (int)((p.M - row0) < MS_ROWS ? (p.M - row0) : MS_ROWS);
        __syncthreads();  // weights are in place (first block); the previous block's buffers are free
        {
            const int K = p.dims[0], Kp = ms_pad4(K);
            const int total = MS_ROWS * Kp;
            for (int base = tid; base < total; base += MS_BATCH * MS_THREADS) {
                float v[MS_BATCH];
#pragma unroll
                for (int u = 0; u < MS_BATCH; ++u) {
                    const int idx = base + u * MS_THREADS;
                    const int r = idx / Kp, k = idx - r * Kp;
                    v[u] = (idx < total && r < rows && k < K) ? Cvt<T>::to_f(x[(row0 + r) * p.lda + k]) : 0.f;
                }
#pragma unroll
                for (int u = 0; u < MS_BATCH; ++u) {
                    const int idx = base + u * MS_THREADS;
                    if (idx < total) act_a[(idx / Kp) * pitch + (idx % Kp)] = v[u];
                }
            }
        }
        __syncthreads();
        float* in = act_a;
        float* nxt = act_b;
        for (int l = 0; l < p.layers; ++l) {
            const int K = p.dims[l], N = p.dims[l + 1], Kp = ms_pad4(K);
            const int npow = ms_pow2(N);
            const int groups = MS_THREADS / npow;                       // >= 2
            const int rpt = MS_ROWS / groups > 0 ? MS_ROWS / groups : 1;  // rows per thread: 1, 2, 4, 8 or 16
            const int n = tid & (npow - 1), g = tid / npow;
            const int r_lo = g * rpt;
            const bool last = (l == p.layers - 1);
            if (n < N && r_lo < MS_ROWS) {
                T* out_rows = last ? out + row0 * p.ldc : nullptr;
                const float* wcol = w_s[l] + n;
                const float bias = b_s[l][n];
                switch (rpt) {
                    case 1: ms_layer<T, 1>(in, nxt, wcol, bias, N, Kp, pitch, r_lo, n, p.act[l], out_rows, p.ldc, rows); break;
                    case 2: ms_layer<T, 2>(in, nxt, wcol, bias, N, Kp, pitch, r_lo, n, p.act[l], out_rows, p.ldc, rows); break;
                    case 4: ms_layer<T, 4>(in, nxt, wcol, bias, N, Kp, pitch, r_lo, n, p.act[l], out_rows, p.ldc, rows); break;
                    case 8: ms_layer<T, 8>(in, nxt, wcol, bias, N, Kp, pitch, r_lo, n, p.act[l], out_rows, p.ldc, rows); break;
                    default: ms_layer<T, 16>(in, nxt, wcol, bias, N, Kp, pitch, r_lo, n, p.act[l], out_rows, p.ldc, rows); break;
                }
            }
            if (!last) {
                // zero the k-padding of the next layer's input (its float4 reads run to the padded width)
                const int Np = ms_pad4(N);
                if (Np > N)
                    for (int idx = tid; idx < MS_ROWS * (Np - N); idx += MS_THREADS)
                        nxt[(idx / (Np - N)) * pitch + N + idx % (Np - N)] = 0.f;
                __syncthreads();
                float* t = in; in = nxt; nxt = t;
            }
        }
    }
}

int64_t smem_floats(const int* dims, int layers) {
    int64_t f = 0;
    int max_dim = dims[0];
    for (int l = 0; l < layers; ++l) {
        f += (int64_t)ms_pad4(dims[l]) * dims[l + 1] + ms_pad4(dims[l + 1]);
        if (dims[l + 1] > max_dim) max_dim = dims[l + 1];
    }
    return f + 2LL * MS_ROWS * (ms_pad4(max_dim) + 4);
}

template <typename T>
int launch_small(const MlpSmallParams& p, cudaStream_t st) {
    const int smem = (int)(smem_floats(p.dims, p.layers) * 4);
    auto kern = mlp_small_kernel<T>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(XG_ERR_LAUNCH, "xg_mlp_small_bias_act: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    const int64_t blocks = (p.M + MS_ROWS - 1) / MS_ROWS;
    int per_sm = (200 * 1024) / (smem + 1024);  // CTAs that fit an SM by shared memory; 8 x 256 threads at most
    per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
    const int64_t cap = (int64_t)per_sm * num_sms();
    kern<<<(unsigned)(blocks < cap ? blocks : cap), MS_THREADS, smem, st>>>(p);
    return check_launch("xg_mlp_small_bias_act");
}

}  // namespace

bool mlp_small_supported(const int64_t* dims, int layers, int dtype) {
    if (!dims || layers < 1 || layers > 3) return false;
    if (dtype != XG_F32 && dtype != XG_BF16 && dtype != XG_F16) return false;
    int64_t weights = 0;
    for (int l = 0; l <= layers; ++l)
        if (dims[l] < 1 || dims[l] > MS_MAX_DIM) return false;
    for (int l = 0; l < layers; ++l) weights += (int64_t)ms_pad4((int)dims[l]) * dims[l + 1];
    return weights <= MS_MAX_WEIGHT_FLOATS;
}

}  // namespace xg

extern "C" int xg_mlp_small_supported(const int64_t* dims, int layers, int dtype) {
    return xg::mlp_small_supported(dims, layers, dtype) ? 1 : 0;
}

extern "C" int xg_mlp_small_bias_act(const void* x, const void* const* w, const void* const* bias, void* out, int64_t M,
                                     const int64_t* dims, int layers, int64_t lda, const int64_t* ldw, int64_t ldc,
                                     const int* act, int weights_kn, int dtype, void* stream) {
    using namespace xg;
    if (!x || !w || !out || !dims || !ldw || !act) return fail(XG_ERR_INVALID_ARG, "xg_mlp_small_bias_act: null pointer");
    if (M < 0) return fail(XG_ERR_INVALID_ARG, "xg_mlp_small_bias_act: negative M");
    if (!mlp_small_supported(dims, layers, dtype))
        return fail(XG_ERR_UNSUPPORTED, "xg_mlp_small_bias_act: 1..3 layers, every width in [1, %d], at most %d weight elements, "
                    "fp32 / bf16 / f16", MS_MAX_DIM, MS_MAX_WEIGHT_FLOATS);
    MlpSmallParams p;
    p.x = x;
    p.out = out;
    p.M = M; p.lda = lda; p.ldc = ldc;
    p.layers = layers;
    p.w_kn = weights_kn;
    p.dims[0] = (int)dims[0];
    for (int l = 0; l < 3; ++l) {
        p.w[l] = l < layers ? w[l] : nullptr;
        p.bias[l] = (l < layers && bias) ? bias[l] : nullptr;
        p.ldw[l] = l < layers ? ldw[l] : 0;
        p.dims[l + 1] = l < layers ? (int)dims[l + 1] : 0;
        p.act[l] = l < layers ? act[l] : 0;
        if (l < layers) {
            if (!w[l]) return fail(XG_ERR_INVALID_ARG, "xg_mlp_small_bias_act: null weight %d", l);
            if (act[l] < XG_ACT_NONE || act[l] > XG_ACT_SIGMOID) return fail(XG_ERR_INVALID_ARG, "xg_mlp_small_bias_act: bad activation %d", act[l]);
            const bool kn = (weights_kn >> l) & 1;
            if (ldw[l] < (kn ? dims[l + 1] : dims[l])) return fail(XG_ERR_INVALID_ARG, "xg_mlp_small_bias_act: ldw[%d] too small", l);
        }
    }
    if (lda < dims[0] || ldc < dims[layers]) return fail(XG_ERR_INVALID_ARG, "xg_mlp_small_bias_act: leading dimension too small");
    if (M == 0) return XG_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (dtype == XG_F32) return launch_small<float>(p, st);
    if (dtype == XG_BF16) return launch_small<__nv_bfloat16>(p, st);
    return launch_small<__half>(p, st);
}
