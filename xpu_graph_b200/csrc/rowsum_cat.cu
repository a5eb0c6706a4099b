// Row reductions written side by side into one matrix:
//   out[b, k*C + c] = sum over r in [r0_k, r1_k) of a_k[b, r, c] * (b_k ? b_k[b, r, c] : 1),   k = 0..n-1
// with a_k / b_k contiguous [*, R_k, C] tensors (a batch stride of 0 broadcasts one [R_k, C] slab over the batch).
// That is slice -> sum(dim 1) -> cat(dim -1) when all a_k are one tensor, sum -> cat for different tensors, and
// mul -> sum -> cat with the second operand. fp32 accumulation; HBM-bound.
//   general kernel: grid.y = segment, a thread owns a 16-byte vector of columns of one batch row and walks the rows
//                   (loads are coalesced across the columns);
//   prefix kernel:  when all segments read the same tensor from the same first row (the slice -> sum -> cat case)
//                   the segments, sorted by their last row, are running sums of one walk: every input row is read
//                   once instead of once per segment.
#include "common.cuh"

namespace xg {
namespace {

constexpr int kMaxSeg = 64;

struct RowSumParams {
    const void* a[kMaxSeg];
    const void* b[kMaxSeg];
    int64_t a_bs[kMaxSeg];  // batch strides in elements (0 = broadcast)
    int64_t b_bs[kMaxSeg];
    int32_t r0[kMaxSeg];
    int32_t r1[kMaxSeg];
    int32_t slot[kMaxSeg];  // output block of the segment
    void* out;
    int64_t out_ld;
    int64_t B;
    int32_t C;
    int32_t n;
};

template <typename T, int V, bool MUL>
__global__ void __launch_bounds__(256) rowsum_cat_kernel(const __grid_constant__ RowSumParams p) {
    const int k = blockIdx.y;
    const int cv = p.C / V;  // column vectors per row
    const T* a = reinterpret_cast<const T*>(p.a[k]);
    const T* b = MUL ? reinterpret_cast<const T*>(p.b[k]) : nullptr;
    const int r0 = p.r0[k], r1 = p.r1[k];
    T* out = reinterpret_cast<T*>(p.out) + (int64_t)p.slot[k] * p.C;
    const int64_t total = p.B * cv;
    for (int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x; e < total; e += (int64_t)gridDim.x * 256) {
        const int64_t bi = e / cv;
        const int c = (int)(e - bi * cv) * V;
        const T* ap = a + bi * p.a_bs[k] + (int64_t)r0 * p.C + c;
        const T* bp = MUL ? b + bi * p.b_bs[k] + (int64_t)r0 * p.C + c : nullptr;
        float acc[V];
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = 0.f;
        int r = r0;
        for (; r + 4 <= r1; r += 4) {  // four rows of loads in flight
            if (V > 1) {
                Vec16<T> va[4], vb[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    va[u] = ld16_stream(ap + (int64_t)u * p.C);
                    if (MUL) vb[u] = ld16_stream(bp + (int64_t)u * p.C);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int i = 0; i < V; ++i)
                        acc[i] += MUL ? Cvt<T>::to_f(va[u].v[i]) * Cvt<T>::to_f(vb[u].v[i]) : Cvt<T>::to_f(va[u].v[i]);
            } else {
                float xa[4], xb[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    xa[u] = Cvt<T>::to_f(ap[(int64_t)u * p.C]);
                    xb[u] = MUL ? Cvt<T>::to_f(bp[(int64_t)u * p.C]) : 1.f;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) acc[0] += MUL ? xa[u] * xb[u] : xa[u];
            }
            ap += 4 * (int64_t)p.C;
            if (MUL) bp += 4 * (int64_t)p.C;
        }
        for (; r < r1; ++r) {
            if (V > 1) {
                const Vec16<T> va = ld16_stream(ap);
                Vec16<T> vb;
                if (MUL) vb = ld16_stream(bp);
#pragma unroll
                for (int i = 0; i < V; ++i) acc[i] += MUL ? Cvt<T>::to_f(va.v[i]) * Cvt<T>::to_f(vb.v[i]) : Cvt<T>::to_f(va.v[i]);
            } else {
                acc[0] += MUL ? Cvt<T>::to_f(ap[0]) * Cvt<T>::to_f(bp[0]) : Cvt<T>::to_f(ap[0]);
            }
            ap += p.C;
            if (MUL) bp += p.C;
        }
        T* op = out + bi * p.out_ld + c;
        if (V > 1) {
            Vec16<T> vo;
#pragma unroll
            for (int i = 0; i < V; ++i) vo.v[i] = Cvt<T>::from_f(acc[i]);
            st16(op, vo);
        } else {
            op[0] = Cvt<T>::from_f(acc[0]);
        }
    }
}

// Segments share a[0], a_bs[0] and r0[0]; r1 ascending (slot[] maps back to the caller's order).
template <typename T, int V>
__global__ void __launch_bounds__(256) rowsum_prefix_kernel(const __grid_constant__ RowSumParams p) {
    const int cv = p.C / V;
    const T* a = reinterpret_cast<const T*>(p.a[0]);
    const int64_t total = p.B * cv;
    for (int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x; e < total; e += (int64_t)gridDim.x * 256) {
        const int64_t bi = e / cv;
        const int c = (int)(e - bi * cv) * V;
        const T* ap = a + bi * p.a_bs[0] + (int64_t)p.r0[0] * p.C + c;
        float acc[V];
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = 0.f;
        int r = p.r0[0];
        for (int k = 0; k < p.n; ++k) {
            const int r1 = p.r1[k];
            for (; r + 4 <= r1; r += 4) {
                if (V > 1) {
                    Vec16<T> va[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) va[u] = ld16_stream(ap + (int64_t)u * p.C);
#pragma unroll
                    for (int u = 0; u < 4; ++u)
#pragma unroll
                        for (int i = 0; i < V; ++i) acc[i] += Cvt<T>::to_f(va[u].v[i]);
                } else {
                    float xa[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) xa[u] = Cvt<T>::to_f(ap[(int64_t)u * p.C]);
#pragma unroll
                    for (int u = 0; u < 4; ++u) acc[0] += xa[u];
                }
                ap += 4 * (int64_t)p.C;
            }
            for (; r < r1; ++r) {
                if (V > 1) {
                    const Vec16<T> va = ld16_stream(ap);
#pragma unroll
                    for (int i = 0; i < V; ++i) acc[i] += Cvt<T>::to_f(va.v[i]);
                } else {
                    acc[0] += Cvt<T>::to_f(ap[0]);
                }
                ap += p.C;
            }
            T* op = reinterpret_cast<T*>(p.out) + bi * p.out_ld + (int64_t)p.slot[k] * p.C + c;
            if (V > 1) {
                Vec16<T> vo;
#pragma unroll
                for (int i = 0; i < V; ++i) vo.v[i] = Cvt<T>::from_f(acc[i]);
                st16(op, vo);
            } else {
                op[0] = Cvt<T>::from_f(acc[0]);
            }
        }
    }
}

template <typename T>
int launch_rowsum(const RowSumParams& p, bool mul, bool prefix, bool vec, cudaStream_t st) {
    constexpr int V = 16 / sizeof(T);
    const int64_t work = (p.B * (vec ? p.C / V : p.C) + 255) / 256;
    const int64_t cap = 32LL * num_sms();
    const unsigned gx = (unsigned)(work < cap ? (work > 0 ? work : 1) : cap);
    if (prefix) {
        if (vec) rowsum_prefix_kernel<T, V><<<gx, 256, 0, st>>>(p);
        else rowsum_prefix_kernel<T, 1><<<gx, 256, 0, st>>>(p);
    } else {
        dim3 grid(gx, (unsigned)p.n);
        if (mul) {
            if (vec) rowsum_cat_kernel<T, V, true><<<grid, 256, 0, st>>>(p);
            else rowsum_cat_kernel<T, 1, true><<<grid, 256, 0, st>>>(p);
        } else {
            if (vec) rowsum_cat_kernel<T, V, false><<<grid, 256, 0, st>>>(p);
            else rowsum_cat_kernel<T, 1, false><<<grid, 256, 0, st>>>(p);
        }
    }
    return check_launch("xg_rowsum_cat");
}

}  // namespace
}  // namespace xg

extern "C" int xg_rowsum_cat(const void* const* a_ptrs, const void* const* b_ptrs, const int64_t* a_batch_strides,
                             const int64_t* b_batch_strides, const int64_t* row_ranges2, int64_t n, int64_t B, int64_t C,
                             void* out, int64_t out_ld, int dtype, void* stream) {
    using namespace xg;
    if (n < 0 || B < 0 || C < 0) return fail(XG_ERR_INVALID_ARG, "xg_rowsum_cat: negative extent");
    const int es = dtype_size(dtype);
    if (es == 0) return fail(XG_ERR_INVALID_ARG, "xg_rowsum_cat: bad dtype %d", dtype);
    if (n == 0 || B == 0 || C == 0) return XG_OK;
    if (!a_ptrs || !a_batch_strides || !row_ranges2 || !out) return fail(XG_ERR_INVALID_ARG, "xg_rowsum_cat: null pointer");
    if (b_ptrs && !b_batch_strides) return fail(XG_ERR_INVALID_ARG, "xg_rowsum_cat: second operands given without strides");
    if (C > 0x7fffffffLL) return fail(XG_ERR_TOO_LARGE, "xg_rowsum_cat: row length %lld", (long long)C);
    if (out_ld < n * C) return fail(XG_ERR_INVALID_ARG, "xg_rowsum_cat: out_ld %lld < n*C", (long long)out_ld);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const bool mul = b_ptrs != nullptr;
    const int V = 16 / es;

    // shared source, shared first row, no second operand -> one walk with running sums
    bool prefix = !mul && n <= kMaxSeg && n > 1;
    for (int64_t k = 0; k < n && prefix; ++k)
        prefix = a_ptrs[k] == a_ptrs[0] && a_batch_strides[k] == a_batch_strides[0] && row_ranges2[2 * k] == row_ranges2[0];

    bool vec = C % V == 0 && aligned16(out) && (out_ld * es) % 16 == 0;
    for (int64_t k = 0; k < n; ++k) {
        const int64_t r0 = row_ranges2[2 * k], r1 = row_ranges2[2 * k + 1];
        if (r0 < 0 || r1 < r0 || r1 > 0x7fffffffLL) return fail(XG_ERR_INVALID_ARG, "xg_rowsum_cat: bad row range of segment %lld", (long long)k);
        if (!a_ptrs[k] && r1 > r0) return fail(XG_ERR_INVALID_ARG, "xg_rowsum_cat: null operand %lld", (long long)k);
        if (mul && !b_ptrs[k] && r1 > r0) return fail(XG_ERR_INVALID_ARG, "xg_rowsum_cat: null second operand %lld", (long long)k);
        vec = vec && aligned16(a_ptrs[k]) && (a_batch_strides[k] * es) % 16 == 0;
        if (mul) vec = vec && aligned16(b_ptrs[k]) && (b_batch_strides[k] * es) % 16 == 0;
    }

    RowSumParams p;
    p.out = out;
    p.out_ld = out_ld;
    p.B = B;
    p.C = (int32_t)C;
    if (prefix) {
        int order[kMaxSeg];
        for (int k = 0; k < n; ++k) order[k] = k;
        for (int i = 1; i < n; ++i) {  // insertion sort by last row (n <= 64)
            const int o = order[i];
            int j = i;
            while (j > 0 && row_ranges2[2 * order[j - 1] + 1] > row_ranges2[2 * o + 1]) {
                order[j] = order[j - 1];
                --j;
            }
            order[j] = o;
        }
        p.n = (int32_t)n;
        for (int k = 0; k < n; ++k) {
            const int o = order[k];
            p.a[k] = a_ptrs[0];
            p.b[k] = nullptr;
            p.a_bs[k] = a_batch_strides[0];
            p.b_bs[k] = 0;
            p.r0[k] = (int32_t)row_ranges2[0];
            p.r1[k] = (int32_t)row_ranges2[2 * o + 1];
            p.slot[k] = o;
        }
        switch (dtype) {
            case XG_F32: return launch_rowsum<float>(p, false, true, vec, st);
            case XG_BF16: return launch_rowsum<__nv_bfloat16>(p, false, true, vec, st);
            default: return launch_rowsum<__half>(p, false, true, vec, st);
        }
    }
    for (int64_t base = 0; base < n; base += kMaxSeg) {
        p.n = 0;
        for (int64_t k = base; k < n && p.n < kMaxSeg; ++k) {
            p.a[p.n] = a_ptrs[k];
            p.b[p.n] = mul ? b_ptrs[k] : nullptr;
            p.a_bs[p.n] = a_batch_strides[k];
            p.b_bs[p.n] = mul ? b_batch_strides[k] : 0;
            p.r0[p.n] = (int32_t)row_ranges2[2 * k];
            p.r1[p.n] = (int32_t)row_ranges2[2 * k + 1];
            p.slot[p.n] = (int32_t)k;
            p.n += 1;
        }
        int rc;
        switch (dtype) {
            case XG_F32: rc = launch_rowsum<float>(p, mul, false, vec, st); break;
            case XG_BF16: rc = launch_rowsum<__nv_bfloat16>(p, mul, false, vec, st); break;
            default: rc = launch_rowsum<__half>(p, mul, false, vec, st); break;
        }
        if (rc != XG_OK) return rc;
    }
    return XG_OK;
}
