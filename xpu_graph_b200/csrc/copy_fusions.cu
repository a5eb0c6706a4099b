// Bit-exact copy fusions: segmented 2-D copy (slice+cat, multi-slice, split, cat/stack, optional
// row mask) and multi-table row gather (embedding lookups fused with where-mask and stack).
//
// Both are single-pass and HBM-bound: every useful byte is read once and written once, in the
// widest unit (up to 16 bytes) that the pointers, strides and lengths allow. The column -> segment
// map is a small look-up table built in shared memory from the segment list, so consecutive
// threads write consecutive output units (coalesced stores; loads are coalesced within a segment).
#include "common.cuh"

namespace xg {
namespace {

constexpr int kMaxSegs = 64;     // segments per launch (kernel parameter space)
constexpr int kLutMax = 8192;    // output units per row per launch (32 KiB of shared memory)
constexpr int kCopyThreads = 256;
constexpr int kCopyUnroll = 4;
constexpr int kGatherRows = 8;    // rows per CTA in the gather kernel

struct SegDesc {
    const char* src;
    char* dst;
    int64_t src_ld;  // bytes
    int64_t dst_ld;  // bytes
    int32_t units;
    int32_t unit_start;
};

struct SegCopyParams {
    SegDesc seg[kMaxSegs];
    int32_t nseg;
    int32_t width;  // total units per row in this launch
    int32_t rows_per_cta;
    int32_t zero_when;
    int64_t rows;
    const uint8_t* mask;
};

template <typename U>
__device__ __forceinline__ U zero_unit() {
    U z;
    memset(&z, 0, sizeof(U));
    return z;
}

template <typename U>
__global__ void __launch_bounds__(kCopyThreads) seg_copy_kernel(const __grid_constant__ SegCopyParams p) {
    __shared__ SegDesc segs[kMaxSegs];
    __shared__ uint32_t lut[kLutMax];
    for (int k = threadIdx.x; k < p.nseg; k += kCopyThreads) segs[k] = p.seg[k];
    __syncthreads();
    for (int k = 0; k < p.nseg; ++k) {
        const int n = segs[k].units, s0 = segs[k].unit_start;
        for (int j = threadIdx.x; j < n; j += kCopyThreads) lut[s0 + j] = ((uint32_t)k << 24) | (uint32_t)j;
    }
    __syncthreads();

    const int64_t r0 = (int64_t)blockIdx.x * p.rows_per_cta;
    const int64_t left = p.rows - r0;
    const int nrows = (int)(left < p.rows_per_cta ? left : p.rows_per_cta);
    const int W = p.width;
    if (W >= 128) {
        // wide rows: walk the columns with stride 256 and take the same column of several rows at once
        // (no index division; 64 bytes of loads in flight per thread: 4 rows of 16-byte units, 8 of narrower ones)
        constexpr int kRowsAtOnce = sizeof(U) >= 16 ? kCopyUnroll : 2 * kCopyUnroll;
        for (int rb = 0; rb < nrows; rb += kRowsAtOnce) {
            for (int c = threadIdx.x; c < W; c += kCopyThreads) {
                const uint32_t e = lut[c];
                const SegDesc& sd = segs[e >> 24];
                const int64_t j = (int64_t)(e & 0xffffffu) * sizeof(U);
                U v[kRowsAtOnce];
#pragma unroll
                for (int k = 0; k < kRowsAtOnce; ++k) {
                    if (rb + k < nrows) {
                        const int64_t row = r0 + rb + k;
                        bool zero = false;
                        if (p.mask != nullptr) zero = ((p.mask[row] != 0) == (p.zero_when != 0));
                        v[k] = zero ? zero_unit<U>() : *reinterpret_cast<const U*>(sd.src + row * sd.src_ld + j);
                    }
                }
#pragma unroll
                for (int k = 0; k < kRowsAtOnce; ++k) {
                    if (rb + k < nrows) *reinterpret_cast<U*>(sd.dst + (r0 + rb + k) * sd.dst_ld + j) = v[k];
                }
            }
        }
        return;
    }
    const int total = nrows * W;  // host keeps rows_per_cta * width below 2^31
    for (int i0 = threadIdx.x; i0 < total; i0 += kCopyThreads * kCopyUnroll) {
        U v[kCopyUnroll];
        U* d[kCopyUnroll];
#pragma unroll
        for (int k = 0; k < kCopyUnroll; ++k) {
            const int i = i0 + k * kCopyThreads;
            if (i < total) {
                const int r = i / W;
                const int c = i - r * W;
                const uint32_t e = lut[c];
                const SegDesc& sd = segs[e >> 24];
                const int64_t j = (int64_t)(e & 0xffffffu) * sizeof(U);
                const int64_t row = r0 + r;
                bool zero = false;
                if (p.mask != nullptr) zero = ((p.mask[row] != 0) == (p.zero_when != 0));
                d[k] = reinterpret_cast<U*>(sd.dst + row * sd.dst_ld + j);
                v[k] = zero ? zero_unit<U>() : *reinterpret_cast<const U*>(sd.src + row * sd.src_ld + j);
            }
        }
#pragma unroll
        for (int k = 0; k < kCopyUnroll; ++k) {
            const int i = i0 + k * kCopyThreads;
            if (i < total) *d[k] = v[k];
        }
    }
}

template <typename U>
int launch_seg_copy(const SegCopyParams& p, cudaStream_t st) {
    const int64_t grid = (p.rows + p.rows_per_cta - 1) / p.rows_per_cta;
    if (grid > 0x7fffffffLL) return fail(XG_ERR_TOO_LARGE, "xg_seg_copy: too many row tiles");
    seg_copy_kernel<U><<<(unsigned)grid, kCopyThreads, 0, st>>>(p);
    return check_launch("xg_seg_copy");
}

int dispatch_seg_copy(int unit, const SegCopyParams& p, cudaStream_t st) {
    switch (unit) {
        case 16: return launch_seg_copy<uint4>(p, st);
        case 8: return launch_seg_copy<uint2>(p, st);
        case 4: return launch_seg_copy<uint32_t>(p, st);
        case 2: return launch_seg_copy<uint16_t>(p, st);
        default: return launch_seg_copy<uint8_t>(p, st);
    }
}

inline int pow2_align(uint64_t v) {  // largest power of two <= 16 dividing v (16 for v == 0)
    int a = 16;
    while (a > 1 && (v % (uint64_t)a) != 0) a >>= 1;
    return a;
}

// ---------------------------------------------------------------------------------------
// multi-table gather
// ---------------------------------------------------------------------------------------
struct GatherParams {
    const char* table[kMaxSegs];
    int64_t table_rows[kMaxSegs];
    int32_t F;
    int32_t f0;             // first field of this launch (offset into idx columns / out columns)
    int32_t units_per_row;  // D * elem_size / sizeof(U)
    int32_t zero_when;
    int64_t rows;
    int64_t row_bytes;  // D * elem_size
    const int64_t* idx;
    int64_t idx_rs, idx_cs;
    const uint8_t* mask;
    char* out;
    int64_t out_ld_bytes;
};

template <typename U>
__global__ void __launch_bounds__(kCopyThreads) gather_rows_kernel(const __grid_constant__ GatherParams p) {
    __shared__ const char* tab[kMaxSegs];
    __shared__ int64_t trows[kMaxSegs];
    for (int k = threadIdx.x; k < p.F; k += kCopyThreads) {
        tab[k] = p.table[k];
        trows[k] = p.table_rows[k];
    }
    __syncthreads();
    // One CTA owns kGatherRows consecutive rows; a thread walks the (field, unit) columns of a row with stride 256
    // and takes the same column of 4 rows at once: 4 index loads, then 4 table loads in flight, 32-bit index math.
    const int upr = p.units_per_row;
    const int per_row = p.F * upr;
    const int64_t r0 = (int64_t)blockIdx.x * kGatherRows;
    for (int rb = 0; rb < kGatherRows; rb += kCopyUnroll) {
        for (int c = threadIdx.x; c < per_row; c += kCopyThreads) {
            const int f = c / upr;
            const int u = c - f * upr;
            int64_t ix[kCopyUnroll];
#pragma unroll
            for (int k = 0; k < kCopyUnroll; ++k) {
                const int64_t r = r0 + rb + k;
                ix[k] = (r < p.rows) ? p.idx[r * p.idx_rs + (int64_t)(p.f0 + f) * p.idx_cs] : -1;
            }
            U v[kCopyUnroll];
#pragma unroll
            for (int k = 0; k < kCopyUnroll; ++k) {
                const int64_t r = r0 + rb + k;
                bool zero = (ix[k] < 0) || (ix[k] >= trows[f]);
                if (r < p.rows && p.mask != nullptr) zero = zero || ((p.mask[r] != 0) == (p.zero_when != 0));
                v[k] = zero ? zero_unit<U>() : reinterpret_cast<const U*>(tab[f] + ix[k] * p.row_bytes)[u];
            }
#pragma unroll
            for (int k = 0; k < kCopyUnroll; ++k) {
                const int64_t r = r0 + rb + k;
                if (r < p.rows)
                    reinterpret_cast<U*>(p.out + r * p.out_ld_bytes + (int64_t)(p.f0 + f) * p.row_bytes)[u] = v[k];
            }
        }
    }
}

template <typename U>
int launch_gather(const GatherParams& p, cudaStream_t st) {
    const int64_t grid = (p.rows + kGatherRows - 1) / kGatherRows;
    if (grid > 0x7fffffffLL) return fail(XG_ERR_TOO_LARGE, "xg_gather_rows: too many tiles");
    gather_rows_kernel<U><<<(unsigned)grid, kCopyThreads, 0, st>>>(p);
    return check_launch("xg_gather_rows");
}

}  // namespace
}  // namespace xg

extern "C" int xg_seg_copy(const void* const* src_ptrs, void* const* dst_ptrs, const int64_t* src_ld_bytes,
                           const int64_t* dst_ld_bytes, const int64_t* len_bytes, int64_t nseg, int64_t rows,
                           const uint8_t* row_mask, int mask_zero_when, void* stream) {
    using namespace xg;
    if (nseg < 0 || rows < 0) return fail(XG_ERR_INVALID_ARG, "xg_seg_copy: negative extent");
    if (nseg == 0 || rows == 0) return XG_OK;
    if (!src_ptrs || !dst_ptrs || !src_ld_bytes || !dst_ld_bytes || !len_bytes)
        return fail(XG_ERR_INVALID_ARG, "xg_seg_copy: null descriptor array");
    uint64_t bits = 0;
    for (int64_t k = 0; k < nseg; ++k) {
        if (len_bytes[k] < 0 || src_ld_bytes[k] < 0 || dst_ld_bytes[k] < 0)
            return fail(XG_ERR_INVALID_ARG, "xg_seg_copy: negative length/stride in segment %lld", (long long)k);
        if (len_bytes[k] == 0) continue;
        if (!src_ptrs[k] || !dst_ptrs[k]) return fail(XG_ERR_INVALID_ARG, "xg_seg_copy: null pointer in segment %lld", (long long)k);
        if (rows > 1 && (src_ld_bytes[k] < len_bytes[k] || dst_ld_bytes[k] < len_bytes[k]))
            return fail(XG_ERR_INVALID_ARG, "xg_seg_copy: stride smaller than length in segment %lld", (long long)k);
        bits |= (uint64_t)reinterpret_cast<uintptr_t>(src_ptrs[k]) | (uint64_t)reinterpret_cast<uintptr_t>(dst_ptrs[k]) |
                (uint64_t)src_ld_bytes[k] | (uint64_t)dst_ld_bytes[k] | (uint64_t)len_bytes[k];
    }
    const int unit = pow2_align(bits & 15u ? (bits & 15u) : 16);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

    SegCopyParams p;
    p.rows = rows;
    p.mask = row_mask;
    p.zero_when = mask_zero_when;
    auto flush = [&]() -> int {
        if (p.nseg == 0) return XG_OK;
        // Rows per CTA: every CTA first copies the segment list out of the (large) parameter block and builds the
        // look-up table, so a CTA should take many rows - about 16 CTAs per SM over the whole launch - but never
        // fewer than a thread takes at once.
        const int64_t min_rows = unit >= 16 ? kCopyUnroll : 2 * kCopyUnroll;
        const int64_t want_ctas = 16LL * num_sms();
        int64_t rpc = (rows + want_ctas - 1) / want_ctas;
        rpc = (rpc + min_rows - 1) / min_rows * min_rows;  // whole groups of the rows a thread takes at once
        if (rpc * p.width > 0x3fffffffLL) rpc = 0x3fffffffLL / p.width;  // the narrow-row path indexes rows * width in 32 bits
        if (rpc < 1) rpc = 1;
        p.rows_per_cta = (int32_t)rpc;
        int rc = dispatch_seg_copy(unit, p, st);
        p.nseg = 0;
        p.width = 0;
        return rc;
    };
    p.nseg = 0;
    p.width = 0;
    for (int64_t k = 0; k < nseg; ++k) {
        int64_t units_left = len_bytes[k] / unit;
        int64_t done = 0;
        while (units_left > 0) {
            if (p.nseg == kMaxSegs || p.width == kLutMax) {
                int rc = flush();
                if (rc != XG_OK) return rc;
            }
            int64_t take = kLutMax - p.width;
            if (take > units_left) take = units_left;
            SegDesc& sd = p.seg[p.nseg];
            sd.src = reinterpret_cast<const char*>(src_ptrs[k]) + done * unit;
            sd.dst = reinterpret_cast<char*>(dst_ptrs[k]) + done * unit;
            sd.src_ld = src_ld_bytes[k];
            sd.dst_ld = dst_ld_bytes[k];
            sd.units = (int32_t)take;
            sd.unit_start = p.width;
            p.nseg += 1;
            p.width += (int32_t)take;
            done += take;
            units_left -= take;
        }
    }
    return flush();
}

extern "C" int xg_gather_rows(const void* const* tables, const int64_t* table_rows, int64_t F, const int64_t* idx,
                              int64_t idx_row_stride, int64_t idx_col_stride, const uint8_t* row_mask,
                              int mask_zero_when, void* out, int64_t rows, int64_t D, int64_t out_ld, int elem_size,
                              void* stream) {
    using namespace xg;
    if (F < 0 || rows < 0 || D < 0) return fail(XG_ERR_INVALID_ARG, "xg_gather_rows: negative extent");
    if (elem_size != 2 && elem_size != 4 && elem_size != 8) return fail(XG_ERR_INVALID_ARG, "xg_gather_rows: elem_size must be 2, 4 or 8");
    if (F == 0 || rows == 0 || D == 0) return XG_OK;
    if (!tables || !table_rows || !idx || !out) return fail(XG_ERR_INVALID_ARG, "xg_gather_rows: null pointer");
    if (out_ld < F * D) return fail(XG_ERR_INVALID_ARG, "xg_gather_rows: out_ld smaller than F*D");
    const int64_t row_bytes = D * elem_size;
    if (row_bytes > 0x7fffffffLL) return fail(XG_ERR_TOO_LARGE, "xg_gather_rows: row too wide");
    uint64_t bits = (uint64_t)reinterpret_cast<uintptr_t>(out) | (uint64_t)(out_ld * elem_size) | (uint64_t)row_bytes;
    for (int64_t f = 0; f < F; ++f) {
        if (!tables[f]) return fail(XG_ERR_INVALID_ARG, "xg_gather_rows: null table %lld", (long long)f);
        if (table_rows[f] < 0) return fail(XG_ERR_INVALID_ARG, "xg_gather_rows: negative table size");
        bits |= (uint64_t)reinterpret_cast<uintptr_t>(tables[f]);
    }
    const int unit = pow2_align(bits & 15u ? (bits & 15u) : 16);
    if (unit < 2) return fail(XG_ERR_UNSUPPORTED, "xg_gather_rows: pointers must be at least 2-byte aligned");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    for (int64_t f0 = 0; f0 < F; f0 += kMaxSegs) {
        GatherParams p;
        p.F = (int32_t)((F - f0) < kMaxSegs ? (F - f0) : kMaxSegs);
        p.f0 = (int32_t)f0;
        for (int k = 0; k < p.F; ++k) {
            p.table[k] = reinterpret_cast<const char*>(tables[f0 + k]);
            p.table_rows[k] = table_rows[f0 + k];
        }
        p.units_per_row = (int32_t)(row_bytes / unit);
        if ((int64_t)p.F * p.units_per_row > 0x3fffffffLL) return fail(XG_ERR_TOO_LARGE, "xg_gather_rows: F * D too large");
        p.zero_when = mask_zero_when;
        p.rows = rows;
        p.row_bytes = row_bytes;
        p.idx = idx;
        p.idx_rs = idx_row_stride;
        p.idx_cs = idx_col_stride;
        p.mask = row_mask;
        p.out = reinterpret_cast<char*>(out);
        p.out_ld_bytes = out_ld * elem_size;
        int rc;
        switch (unit) {
            case 16: rc = launch_gather<uint4>(p, st); break;
            case 8: rc = launch_gather<uint2>(p, st); break;
            case 4: rc = launch_gather<uint32_t>(p, st); break;
            default: rc = launch_gather<uint16_t>(p, st); break;
        }
        if (rc != XG_OK) return rc;
    }
    return XG_OK;
}
