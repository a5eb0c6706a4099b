// Dense layer on the 5th-generation tensor cores: out = act(A @ W^T + bias + residual), 16-bit inputs,
// fp32 accumulation in TMEM, epilogue fused into the store.
//
// Persistent kernel, one CTA per SM, warp-specialised:
//   warp 0      : TMA producer  - streams [128 x 64] A tiles and [BN x 64] W tiles (128-byte swizzle)
//                 through a STAGES-deep shared-memory ring, one mbarrier pair (full/empty) per stage;
//   warp 1      : MMA issuer    - one elected thread issues tcgen05.mma (128 x BN x 16) straight from
//                 shared memory into one of two TMEM accumulator buffers; tcgen05.commit releases the
//                 ring stage and, after the last k-block, publishes the accumulator;
//   warps 2..5  : epilogue      - tcgen05.ld the accumulator (each warp owns its 32-lane TMEM quadrant),
//                 add bias / residual, apply the activation, convert and store, then hand the TMEM
//                 buffer back. The second accumulator buffer lets tile i's epilogue overlap tile i+1's
//                 main loop.
// Tiles are visited in groups of 16 row-blocks so that the ~148 tiles in flight share A and W tiles in L2.
// Every TMA load is issued by the CTA that consumes it (no cluster multicast anywhere).
#include "common.cuh"
#include "sm100_ptx.cuh"

#include <cstdlib>
#include <mutex>
#include <type_traits>

namespace xg {

// Optional rotary-embedding epilogue: out[row, h*D + j] gets the rotate-half RoPE of the accumulator row at
// position (row % S), with cos/sin tables [S, D] of the output dtype.
struct GemmExtras {
    const void* rope_cos = nullptr;
    const void* rope_sin = nullptr;
    int64_t rope_S = 0;
    int rope_D = 0;
};

int gemm_tc_entry(const void* A, const void* B, const void* bias, const void* residual, void* out, int64_t M, int64_t N,
                  int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr, int trans_b, int act, int dtype,
                  void* workspace, int64_t ws_bytes, cudaStream_t st, bool force_split = false,
                  const GemmExtras* extras = nullptr);

bool plan_ksplit(int64_t M, int64_t N, int64_t K, int dtype, int* S_out, int* tn_out);
int gemm_tc_ksplit_entry(const void* A, const void* W, const void* bias, const void* residual, void* out, int64_t M,
                         int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int act, int dtype, int S,
                         int tn, cudaStream_t st);

struct GemmPlan {
    int bn;      // tile width: 64, 128 or 256
    int splits;  // split-K factor (1 = none)
};

// ---- tensor-map helpers (host) ----------------------------------------------------------------
PFN_encodeTiled get_encode_tiled() {
    static PFN_encodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, []() {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_encodeTiled>(p);
        else
            cudaGetLastError();
    });
    return fn;
}

bool make_tmap_2d_16bit(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                        uint32_t box_rows, uint32_t box_cols, bool is_bf16) {
    PFN_encodeTiled enc = get_encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                     const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// [batch][rows][cols] with row stride ld and batch stride bs (elements): dims (cols, rows, batch), box (box_cols, box_rows, 1).
bool make_tmap_3d_16bit(CUtensorMap* out, const void* base, uint64_t batch, uint64_t rows, uint64_t cols, uint64_t ld,
                        uint64_t bs, uint32_t box_rows, uint32_t box_cols, bool is_bf16) {
    PFN_encodeTiled enc = get_encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[3] = {cols, rows, batch};
    cuuint64_t strides[2] = {ld * 2, bs * 2};
    cuuint32_t box[3] = {box_cols, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(out, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                     const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

bool make_tmap_bhsd_16bit(CUtensorMap* out, const void* base, uint64_t B, uint64_t H, uint64_t S, uint64_t D,
                          uint64_t stride_b, uint64_t stride_h, uint64_t stride_s, uint32_t box_rows, bool is_bf16) {
    PFN_encodeTiled enc = get_encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[4] = {D, S, H, B};
    // A stride of a size-1 dimension is never used for addressing but must still be a valid multiple of 16 bytes.
    auto fix = [&](uint64_t st, uint64_t extent) -> cuuint64_t { return (extent == 1 || st == 0) ? D * 2 : st * 2; };
    cuuint64_t strides[3] = {fix(stride_s, S), fix(stride_h, H), fix(stride_b, B)};
    cuuint32_t box[4] = {64, box_rows, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(out, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                     const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Device-side status word: non-zero after a bounded wait expired inside a tcgen05 kernel.
__device__ unsigned int g_tc_status[4];

namespace {

constexpr int BM = 128;
constexpr int BK = 64;       // 64 x 16-bit = one 128-byte swizzled row
constexpr int UMMA_K = 16;
constexpr int kGemmThreads = 192;
constexpr int GROUP_M = 16;

// Scalar kernel parameters. The struct is kept at 128 bytes: next to three tensor maps the parameter block is then
// exactly 512 bytes. (Measured: 16 bytes more cost the CTA-pair kernel 5 % of its throughput and 30 % with a residual
// epilogue - the same source with a padded struct reproduces it - so the fields of the mutually exclusive variants
// share storage.)
enum GemmMode : int {
    kModePlain = 0,      // 16-bit output; split-K when splits > 1 (split.partial)
    kModeRope = 1,       // rotary-embedding epilogue (rope.*)
    kModeF32 = 2,        // fp32 problem from bf16 planes: out, bias and residual are fp32 (f32.*)
    kModeF32Planes = 3,  // same, out is the next layer's operand: three bf16 planes per row ([M, 3 * out_kp], columns
                         // N..out_kp-1 zero), bias fp32, no residual
    kModeBatch = 4,      // batched (single-CTA kernel): 3-D tensor maps, work units (entry, tile) (batch.*)
};

struct GemmParams {
    void* out;
    const void* bias;
    const void* residual;
    int64_t M, N, K, ldc, ldr;
    int act;
    int vec_ok;       // out (and residual) rows are 16-byte addressable
    int bias_vec_ok;  // bias pointer 16-byte aligned
    int num_m_blocks, num_n_blocks, num_k_blocks;
    int splits;  // > 1: split-K, every (tile, split) unit writes raw fp32 accumulators to split.partial
    int mode;    // GemmMode
    union {
        struct {
            float* partial;  // [splits][M][N] fp32 workspace
        } split;
        struct {
            const void* cos;
            const void* sin;
            int64_t S;
            int D;
        } rope;
        struct {
            // Operands made of K-segments laid side by side (the three bf16 planes of an fp32 matrix): the k-blocks run
            // over `seg_blocks`-long segment PAIRS, pair i reading segment (seg_a >> 4i) & 15 of A against
            // (seg_b >> 4i) & 15 of W.
            int seg_blocks;
            uint32_t seg_a, seg_b;
            int pad_;
            int64_t out_kp;
        } f32;
        struct {
            int64_t bs_out, bs_bias, bs_res;  // elements per entry
            int count;
        } batch;
    };
};
static_assert(sizeof(GemmParams) == 128, "GemmParams must stay at 128 bytes (512-byte kernel parameter block)");

__host__ __device__ __forceinline__ int f32_mode_of(const GemmParams& p) {
    return p.mode == kModeF32 ? 1 : (p.mode == kModeF32Planes ? 2 : 0);
}
__host__ __device__ __forceinline__ int batch_of(const GemmParams& p) { return p.mode == kModeBatch ? p.batch.count : 1; }

// Element offsets along K of k-block kb in the A and the W tensor map.
__device__ __forceinline__ void kblock_coords(const GemmParams& p, int kb, int& ka, int& kw) {
    if (f32_mode_of(p) == 0) {
        ka = kw = kb * BK;
        return;
    }
    const int sb = p.f32.seg_blocks;
    const int pair = kb / sb, kk = kb - pair * sb;
    ka = ((int)((p.f32.seg_a >> (4 * pair)) & 15u) * sb + kk) * BK;
    kw = ((int)((p.f32.seg_b >> (4 * pair)) & 15u) * sb + kk) * BK;
}

// k-block range of split s of `splits` over nkb blocks (balanced, every split non-empty when splits <= nkb)
__device__ __forceinline__ void split_range(int s, int splits, int nkb, int& kb0, int& kb1) {
    const int base = nkb / splits, rem = nkb % splits;
    kb0 = s * base + (s < rem ? s : rem);
    kb1 = kb0 + base + (s < rem ? 1 : 0);
}

template <int BN>
struct GemmCfg {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
    static constexpr int TMEM_COLS = 2 * BN;  // two accumulator buffers; 128, 256 or 512 (powers of two)
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

__device__ __forceinline__ float apply_act(float v, int act) {
    switch (act) {
        case XG_ACT_GELU: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
        case XG_ACT_RELU: return v > 0.f ? v : 0.f;
        case XG_ACT_SILU: return __fdividef(v, 1.0f + __expf(-v));
        case XG_ACT_SIGMOID: return __fdividef(1.0f, 1.0f + __expf(-v));
        default: return v;
    }
}

// ... for results that are rounded to a 16-bit type
template <typename T>
__device__ __forceinline__ float apply_act_out(float v, int act) {
    if (sizeof(T) == 2 && act == XG_ACT_GELU) return gelu_erf_16bit(v);
    return apply_act(v, act);
}

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& mb, int& nb) {
    const int per_group = GROUP_M * num_n;
    const int g = t / per_group;
    const int first_m = g * GROUP_M;
    const int gsz = (num_m - first_m) < GROUP_M ? (num_m - first_m) : GROUP_M;
    const int in_g = t - g * per_group;
    mb = first_m + in_g % gsz;
    nb = in_g / gsz;
}

// One warp's share of a finished accumulator tile: its 32 TMEM lanes (rows), all output columns of the tile in
// chunks of 32: TMEM -> registers -> (+bias, +residual, activation | SwiGLU | raw split-K partials) -> global.
// Warp-collective (tcgen05.ld): all 32 lanes call it, rows past M only skip the stores.
template <typename T, int BN, bool SWIGLU>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, uint32_t tmem_base, int acc, int quad, int64_t row,
                                              bool row_ok, int nb, int split, int entry = 0) {
    constexpr int OUT_BN = SWIGLU ? BN / 2 : BN;
    T* out = reinterpret_cast<T*>(p.out);
    const T* bias = reinterpret_cast<const T*>(p.bias);
    const T* resid = reinterpret_cast<const T*>(p.residual);
    if (p.mode == kModeBatch) {
        out += entry * p.batch.bs_out;
        if (bias) bias += entry * p.batch.bs_bias;
        if (resid) resid += entry * p.batch.bs_res;
    }
    const int f32_mode = f32_mode_of(p);
    if (!SWIGLU && p.mode == kModeRope) {
        // Rotary epilogue: the two halves of a head (columns j and j + D/2) meet in one thread, which owns the whole
        // row of the tile: read the two 32-column chunks that are D/2 apart, rotate, store both. The host guarantees
        // N % D == 0, D in {64, 128}, 16-byte addressable rows and tables.
        const int D = p.rope.D, half_chunks = D / 64;  // chunks of 32 per half head: 1 (D = 64) or 2 (D = 128)
        const int64_t pos = row_ok ? row % p.rope.S : 0;
        const T* cosr = reinterpret_cast<const T*>(p.rope.cos) + pos * D;
        const T* sinr = reinterpret_cast<const T*>(p.rope.sin) + pos * D;
#pragma unroll 1
        for (int c = 0; c < OUT_BN / 32; ++c) {
            const int in_head = c % (2 * half_chunks);
            if (in_head >= half_chunks) continue;  // second half: handled with its partner below
            const int64_t col0 = (int64_t)nb * OUT_BN + c * 32;
            if (col0 >= p.N) break;
            const int c2 = c + half_chunks;
            uint32_t r1[32], r2[32];
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN);
            ptx::tmem_ld_32x32(taddr + (uint32_t)(c * 32), r1);
            ptx::tmem_ld_32x32(taddr + (uint32_t)(c2 * 32), r2);
            ptx::tmem_ld_wait();
            if (row_ok) {
                const int j0 = (c % (2 * half_chunks)) * 32;  // column inside the head of the first half
                T* o1 = out + row * p.ldc + col0;
                T* o2 = o1 + D / 2;
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    const Vec16<T> c1 = ld16(cosr + j0 + i), s1 = ld16(sinr + j0 + i);
                    const Vec16<T> cc2 = ld16(cosr + j0 + D / 2 + i), s2 = ld16(sinr + j0 + D / 2 + i);
                    Vec16<T> y1, y2;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        // the projection result is rounded to the tensor dtype first, as the un-fused graph does
                        const float a = Cvt<T>::to_f(Cvt<T>::from_f(__uint_as_float(r1[i + j])));
                        const float b = Cvt<T>::to_f(Cvt<T>::from_f(__uint_as_float(r2[i + j])));
                        y1.v[j] = Cvt<T>::from_f(a * Cvt<T>::to_f(c1.v[j]) - b * Cvt<T>::to_f(s1.v[j]));
                        y2.v[j] = Cvt<T>::from_f(b * Cvt<T>::to_f(cc2.v[j]) + a * Cvt<T>::to_f(s2.v[j]));
                    }
                    st16(o1 + i, y1);
                    st16(o2 + i, y2);
                }
            }
        }
        return;
    }
#pragma unroll 1
    for (int c = 0; c < OUT_BN / 32; ++c) {
        const int64_t col0 = (int64_t)nb * OUT_BN + c * 32;
        if (col0 >= (f32_mode == 2 ? p.f32.out_kp : p.N)) break;  // warp-uniform
        uint32_t r[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN + c * 32);
        ptx::tmem_ld_32x32(taddr, r);
        ptx::tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        if (SWIGLU) {
            ptx::tmem_ld_32x32(taddr + (uint32_t)(BN / 2), r);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __fdividef(v[i], 1.0f + __expf(-v[i])) * __uint_as_float(r[i]);
        }
        const bool full = (col0 + 32 <= p.N);
        if (f32_mode != 0) {
            const float* biasf = reinterpret_cast<const float*>(p.bias);
            if (biasf != nullptr) {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (col0 + i < p.N) v[i] += biasf[col0 + i];
            }
            if (!row_ok) continue;
            if (f32_mode == 1) {
                const float* rr = p.residual ? reinterpret_cast<const float*>(p.residual) + row * p.ldr + col0 : nullptr;
                float* orow = reinterpret_cast<float*>(p.out) + row * p.ldc + col0;
                if (full && p.vec_ok) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                        if (rr != nullptr) {
                            const float4 r4 = *reinterpret_cast<const float4*>(rr + i);
                            o.x += r4.x; o.y += r4.y; o.z += r4.z; o.w += r4.w;
                        }
                        o.x = apply_act(o.x, p.act); o.y = apply_act(o.y, p.act);
                        o.z = apply_act(o.z, p.act); o.w = apply_act(o.w, p.act);
                        *reinterpret_cast<float4*>(orow + i) = o;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (col0 + i < p.N) orow[i] = apply_act(v[i] + (rr != nullptr ? rr[i] : 0.f), p.act);
                }
            } else {
                // next layer's operand: x = x0 + x1 + x2 in bf16, plane s at columns [s * out_kp, s * out_kp + out_kp)
                __nv_bfloat16* o3 = reinterpret_cast<__nv_bfloat16*>(p.out) + row * (3 * p.f32.out_kp) + col0;
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    if (col0 + i >= p.f32.out_kp) break;
                    Vec16<__nv_bfloat16> q0, q1, q2;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float x = (col0 + i + j < p.N) ? apply_act(v[i + j], p.act) : 0.f;
                        q0.v[j] = __float2bfloat16_rn(x);
                        const float r1 = x - __bfloat162float(q0.v[j]);
                        q1.v[j] = __float2bfloat16_rn(r1);
                        q2.v[j] = __float2bfloat16_rn(r1 - __bfloat162float(q1.v[j]));
                    }
                    st16(o3 + i, q0);
                    st16(o3 + p.f32.out_kp + i, q1);
                    st16(o3 + 2 * p.f32.out_kp + i, q2);
                }
            }
            continue;
        }
        if (p.splits > 1) {
            // split-K: raw fp32 partial sums; bias / residual / activation happen in the reduce kernel
            if (row_ok) {
                float* prow = p.split.partial + ((int64_t)split * p.M + row) * p.N + col0;
                if (full && (p.N & 3) == 0) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4*>(prow + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (col0 + i < p.N) prow[i] = v[i];
                }
            }
            continue;
        }
        if (bias != nullptr) {
            if (full && p.bias_vec_ok) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    const Vec16<T> bv = ld16(bias + col0 + i);
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[i + j] += Cvt<T>::to_f(bv.v[j]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (col0 + i < p.N) v[i] += Cvt<T>::to_f(bias[col0 + i]);
            }
        }
        if (row_ok) {
            if (full && p.vec_ok) {
                if (resid != nullptr) {
                    const T* rr = resid + row * p.ldr + col0;
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        const Vec16<T> rv = ld16_stream(rr + i);
#pragma unroll
                        for (int j = 0; j < 8; ++j) v[i + j] += Cvt<T>::to_f(rv.v[j]);
                    }
                }
                T* orow = out + row * p.ldc + col0;
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    Vec16<T> ov;
#pragma unroll
                    for (int j = 0; j < 8; ++j) ov.v[j] = Cvt<T>::from_f(apply_act_out<T>(v[i + j], p.act));
                    st16(orow + i, ov);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (col0 + i < p.N) {
                        float a = v[i];
                        if (resid != nullptr) a += Cvt<T>::to_f(resid[row * p.ldr + col0 + i]);
                        out[row * p.ldc + col0 + i] = Cvt<T>::from_f(apply_act_out<T>(a, p.act));
                    }
                }
            }
        }
    }
}

// SWIGLU: the W tile is [gate rows ; up rows] (BN/2 each, two TMA loads), so accumulator columns
// [0, BN/2) hold A @ Wg^T and [BN/2, BN) hold A @ Wu^T; the epilogue writes silu(gate) * up, BN/2 wide.
// B_MN: W is given as [K, N] row-major (N contiguous): its tiles are loaded as BN/64 boxes of [64 k x 64 n] and
// consumed MN-major (the layout TMA leaves: rows = k, 128-byte rows of n), so no transpose is ever materialised.
template <typename T, int BN, bool SWIGLU, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_b2, const GemmParams p) {
    constexpr int OUT_BN = SWIGLU ? BN / 2 : BN;  // output columns per tile
    using Cfg = GemmCfg<BN>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: required by the 128-byte swizzle pattern shared by TMA and the MMA descriptors.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * Cfg::A_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
    uint64_t* full_bar = bars;                    // [STAGES]
    uint64_t* empty_bar = bars + STAGES;          // [STAGES]
    uint64_t* tmem_full = bars + 2 * STAGES;      // [2]
    uint64_t* tmem_empty = bars + 2 * STAGES + 2; // [2]
    uint64_t* drain_bar = bars + 2 * STAGES + 4;  // [1]
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 5);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(&tmem_full[a], 1);
            ptx::mbar_init(&tmem_empty[a], 4);
        }
        ptx::mbar_init(drain_bar, 1);
        *abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::fence_proxy_async();
    }
    if (warp == 1) ptx::tmem_alloc(tmem_base_slot, Cfg::TMEM_COLS);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    const int tiles_per_entry = p.num_m_blocks * p.num_n_blocks;
    const int num_tiles = tiles_per_entry * p.splits * batch_of(p);  // work units: (batch entry, tile, split); batch > 1 has no splits
    const int nkb = p.num_k_blocks;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (ptx::elect_one()) {
            ptx::prefetch_tensormap(&tmap_a);
            ptx::prefetch_tensormap(&tmap_b);
            if (SWIGLU) ptx::prefetch_tensormap(&tmap_b2);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t armed = 0;                 // stages with a load this thread issued
            uint32_t armed_phase = 0;           // parity of that load's phase, one bit per stage
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                int mb, nb, kb0, kb1;
                const int unit = t / p.splits, entry = unit / tiles_per_entry;
                tile_coords(unit - entry * tiles_per_entry, p.num_m_blocks, p.num_n_blocks, mb, nb);
                split_range(t % p.splits, p.splits, nkb, kb0, kb1);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!ptx::mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
                    ptx::mbar_arrive_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
                    int ka, kw;
                    kblock_coords(p, kb, ka, kw);
                    if (p.mode == kModeBatch) {  // 3-D maps (k, row, entry); plain and [K, N] weights only
                        ptx::tma_load_3d(smem_a + stage * Cfg::A_BYTES, &tmap_a, &full_bar[stage], ka, mb * BM, entry);
                        if (B_MN) {
#pragma unroll
                            for (int j = 0; j < BN / 64; ++j)
                                ptx::tma_load_3d(smem_b + stage * Cfg::B_BYTES + j * (BK * 128), &tmap_b, &full_bar[stage],
                                                 nb * BN + j * 64, kb * BK, entry);
                        } else {
                            ptx::tma_load_3d(smem_b + stage * Cfg::B_BYTES, &tmap_b, &full_bar[stage], kw, nb * BN, entry);
                        }
                        armed |= 1u << stage;
                        armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
                        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                        continue;
                    }
                    ptx::tma_load_2d(smem_a + stage * Cfg::A_BYTES, &tmap_a, &full_bar[stage], ka, mb * BM);
                    if (SWIGLU) {
                        ptx::tma_load_2d(smem_b + stage * Cfg::B_BYTES, &tmap_b, &full_bar[stage], kb * BK, nb * OUT_BN);
                        ptx::tma_load_2d(smem_b + stage * Cfg::B_BYTES + Cfg::B_BYTES / 2, &tmap_b2, &full_bar[stage],
                                         kb * BK, nb * OUT_BN);
                    } else if (B_MN) {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            ptx::tma_load_2d(smem_b + stage * Cfg::B_BYTES + j * (BK * 128), &tmap_b, &full_bar[stage],
                                             nb * BN + j * 64, kb * BK);
                    } else {
                        ptx::tma_load_2d(smem_b + stage * Cfg::B_BYTES, &tmap_b, &full_bar[stage], kw, nb * BN);
                    }
                    armed |= 1u << stage;
                    armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                // Unwinding: let this thread's own copies land before the CTA gives up its shared memory.
                atomicOr(&g_tc_status[0], 1u);
                for (int s = 0; s < STAGES; ++s) {
                    if (armed & (1u << s)) {
                        const uint64_t t0 = ptx::globaltimer_ns();
                        while (!ptx::mbar_try_wait(&full_bar[s], (armed_phase >> s) & 1u)) {
                            if (ptx::globaltimer_ns() - t0 > ptx::kWaitLimitNs) break;
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::make_idesc_f16(std::is_same<T, __nv_bfloat16>::value ? 1 : 0, BM, BN, B_MN ? 1 : 0);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                if (!ptx::mbar_wait_bounded(&tmem_empty[acc], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                ptx::tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                int kb0, kb1;
                split_range(t % p.splits, p.splits, nkb, kb0, kb1);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!ptx::mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
                    ptx::tc_fence_after();
                    const uint32_t a_addr = ptx::smem_u32(smem_a + stage * Cfg::A_BYTES);
                    const uint32_t b_addr = ptx::smem_u32(smem_b + stage * Cfg::B_BYTES);
                    const uint64_t da = ptx::make_kmajor_sw128_desc(a_addr);
                    const uint64_t db = B_MN ? ptx::make_mnmajor_sw128_desc(b_addr, BK * 128) : ptx::make_kmajor_sw128_desc(b_addr);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // K-major: +32 bytes per 16-element K step; MN-major: +16 rows of 128 bytes
                        // (both in the descriptor's 16-byte address units)
                        const uint64_t db_k = db + (uint64_t)(B_MN ? k * 128 : k * 2);
                        ptx::mma_f16_ss(tmem_d, da + (uint64_t)(k * 2), db_k, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
                    }
                    ptx::tc_commit(&empty_bar[stage]);  // stage reusable once these MMAs have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                ptx::tc_commit(&tmem_full[acc]);  // accumulator complete
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
            if (!ok) {
                atomicOr(&g_tc_status[0], 2u);
                // Let the MMAs already issued finish before TMEM is released.
                ptx::tc_commit(drain_bar);
                const uint64_t t0 = ptx::globaltimer_ns();
                while (!ptx::mbar_try_wait(drain_bar, 0)) {
                    if (ptx::globaltimer_ns() - t0 > ptx::kWaitLimitNs) break;
                }
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------
        const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad + 32) belong to this warp
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        T* out = reinterpret_cast<T*>(p.out);
        const T* bias = reinterpret_cast<const T*>(p.bias);
        const T* resid = reinterpret_cast<const T*>(p.residual);
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            int mb, nb;
            const int unit = t / p.splits, entry = unit / tiles_per_entry;
            tile_coords(unit - entry * tiles_per_entry, p.num_m_blocks, p.num_n_blocks, mb, nb);
            // warp-uniform result: the TMEM loads below are warp-collective
            if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(&tmem_full[acc], acc_phase, abort_flag))) { ok = false; break; }
            ptx::tc_fence_after();
            const int64_t row = (int64_t)mb * BM + quad * 32 + lane;
            const bool row_ok = row < p.M;
            epilogue_tile<T, BN, SWIGLU>(p, tmem_base, acc, quad, row, row_ok, nb, t % p.splits, entry);
            // All of this warp's TMEM reads are complete (wait::ld above): return the buffer.
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&tmem_empty[acc]);
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
        if (!ok && lane == 0) atomicOr(&g_tc_status[0], 4u);
    }

    // ------------------------------ teardown --------------------------------------
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------------------
// CTA-pair variant (cluster of 2, tcgen05 cta_group::2) for large problems.
// A pair owns a 256 x 256 output tile: CTA r loads A rows [r*128, r*128+128) and W rows [r*128, r*128+128) of the tile
// (32 KiB per stage instead of 48, so 6 stages fit and each SM pulls a third less through L2 per FLOP); one thread of
// the leader CTA issues 256 x 256 x 16 MMAs that span both SMs; each CTA's TMEM holds its 128 rows x 256 columns
// (two accumulator buffers), and each CTA's epilogue warps store their own rows.
// Barriers: "full" lives in the leader only and counts the bytes of both CTAs' loads; "empty" and "accumulator full"
// exist in both CTAs and are signalled by the leader's tcgen05.commit (one commit per CTA, no multicast);
// "accumulator empty" lives in the leader and collects the 8 epilogue warps of the pair.
// ---------------------------------------------------------------------------------------------------------
constexpr int PAIR_BN = 256;
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_STAGE_BYTES = (BM + PAIR_BN / 2) * BK * 2;  // per CTA: A tile + half of the W tile = 32 KiB
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 256;

template <typename T, bool SWIGLU>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_b2, const GemmParams p) {
    constexpr int BN = PAIR_BN;
    constexpr int OUT_BN = SWIGLU ? BN / 2 : BN;
    constexpr int STAGES = PAIR_STAGES;
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = (BN / 2) * BK * 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * A_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * PAIR_STAGE_BYTES);
    uint64_t* full_bar = bars;                     // [STAGES]  (used in the leader)
    uint64_t* empty_bar = bars + STAGES;           // [STAGES]  (each CTA its own)
    uint64_t* tmem_full = bars + 2 * STAGES;       // [2]       (each CTA its own)
    uint64_t* tmem_empty = bars + 2 * STAGES + 2;  // [2]       (used in the leader, 8 arrivals)
    uint64_t* drain_bar = bars + 2 * STAGES + 4;   // [1]
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 5);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();  // 0 = leader
    const int pair = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(&tmem_full[a], 1);
            ptx::mbar_init(&tmem_empty[a], 8);
        }
        ptx::mbar_init(drain_bar, 1);
        *abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::fence_proxy_async();
    }
    if (warp == 1) ptx::tmem_alloc_pair(tmem_base_slot, 2 * BN);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();  // both CTAs' barriers are initialised before anyone signals across the pair
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    const int num_tiles = p.num_m_blocks * p.num_n_blocks;  // 256-row blocks x OUT_BN-column blocks
    const int nkb = p.num_k_blocks;

    if (warp == 0) {
        // ------------------------------ TMA producer (both CTAs) ------------------------------
        if (ptx::elect_one()) {
            ptx::prefetch_tensormap(&tmap_a);
            ptx::prefetch_tensormap(&tmap_b);
            if (SWIGLU) ptx::prefetch_tensormap(&tmap_b2);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int issued = 0;
            for (int t = pair; t < num_tiles && ok; t += num_pairs) {
                int mb, nb;
                tile_coords(t, p.num_m_blocks, p.num_n_blocks, mb, nb);
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!ptx::mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
                    if (rank == 0) ptx::mbar_arrive_expect_tx(&full_bar[stage], 2 * PAIR_STAGE_BYTES);
                    const uint32_t full_leader = ptx::map_to_cta(ptx::smem_u32(&full_bar[stage]), 0);
                    int ka, kw;
                    kblock_coords(p, kb, ka, kw);
                    ptx::tma_load_2d_pair(smem_a + stage * A_BYTES, &tmap_a, full_leader, ka, mb * 256 + (int)rank * BM);
                    if (SWIGLU)  // leader: gate rows, partner: up rows of the same 128 output columns
                        ptx::tma_load_2d_pair(smem_b + stage * B_BYTES, rank == 0 ? &tmap_b : &tmap_b2, full_leader, kw,
                                              nb * OUT_BN);
                    else
                        ptx::tma_load_2d_pair(smem_b + stage * B_BYTES, &tmap_b, full_leader, kw,
                                              nb * BN + (int)rank * (BN / 2));
                    ++issued;
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) atomicOr(&g_tc_status[0], 1u);
            (void)issued;
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (leader CTA only) --------------------------------
        if (rank == 0 && ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::make_idesc_f16(std::is_same<T, __nv_bfloat16>::value ? 1 : 0, 256, BN, 0);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int t = pair; t < num_tiles && ok; t += num_pairs) {
                if (!ptx::mbar_wait_bounded(&tmem_empty[acc], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                ptx::tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!ptx::mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
                    ptx::tc_fence_after();
                    const uint64_t da = ptx::make_kmajor_sw128_desc(ptx::smem_u32(smem_a + stage * A_BYTES));
                    const uint64_t db = ptx::make_kmajor_sw128_desc(ptx::smem_u32(smem_b + stage * B_BYTES));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        ptx::mma_f16_ss_pair(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0 ? 1u : 0u);
                    // the stage is free in both CTAs once these MMAs have read it
                    const uint32_t e = ptx::smem_u32(&empty_bar[stage]);
                    ptx::tc_commit_pair(ptx::map_to_cta(e, 0));
                    ptx::tc_commit_pair(ptx::map_to_cta(e, 1));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                const uint32_t f = ptx::smem_u32(&tmem_full[acc]);
                ptx::tc_commit_pair(ptx::map_to_cta(f, 0));
                ptx::tc_commit_pair(ptx::map_to_cta(f, 1));
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
            if (!ok) {
                atomicOr(&g_tc_status[0], 2u);
                ptx::tc_commit_pair(ptx::map_to_cta(ptx::smem_u32(drain_bar), 0));
                const uint64_t t0 = ptx::globaltimer_ns();
                while (!ptx::mbar_try_wait(drain_bar, 0)) {
                    if (ptx::globaltimer_ns() - t0 > ptx::kWaitLimitNs) break;
                }
            }
        }
    } else {
        // ------------------------------ epilogue (both CTAs) ----------------------------------
        const int quad = warp & 3;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int t = pair; t < num_tiles && ok; t += num_pairs) {
            int mb, nb;
            tile_coords(t, p.num_m_blocks, p.num_n_blocks, mb, nb);
            if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(&tmem_full[acc], acc_phase, abort_flag))) { ok = false; break; }
            ptx::tc_fence_after();
            const int64_t row = (int64_t)mb * 256 + (int64_t)rank * BM + quad * 32 + lane;
            epilogue_tile<T, BN, SWIGLU>(p, tmem_base, acc, quad, row, row < p.M, nb, 0);
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&tmem_empty[acc]), 0));
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
        if (!ok && lane == 0) atomicOr(&g_tc_status[0], 4u);
    }

    // ------------------------------ teardown --------------------------------------
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();  // neither CTA leaves (or frees TMEM) while its partner may still touch it
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, 2 * BN);
    }
}

template <typename T, bool SWIGLU>
int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const GemmParams& p,
                     cudaStream_t st) {
    auto kern = gemm_tc_pair_kernel<T, SWIGLU>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(XG_ERR_LAUNCH, "xg_gemm_bias_act: cannot reserve %d bytes of shared memory: %s", PAIR_SMEM_BYTES,
                    cudaGetErrorString(e));
    }
    const int tiles = p.num_m_blocks * p.num_n_blocks;
    // as many pairs as can be resident at once (a pair needs two free SMs of one TPC)
    static thread_local int max_pairs_cached[2] = {0, 0};
    int& max_pairs = max_pairs_cached[SWIGLU ? 1 : 0];
    if (max_pairs == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * (unsigned)(num_sms() / 2));
        cfg.blockDim = dim3(kGemmThreads);
        cfg.dynamicSmemBytes = PAIR_SMEM_BYTES;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = num_sms() / 2;
        }
        max_pairs = n < num_sms() / 2 ? n : num_sms() / 2;
    }
    const int pairs = tiles < max_pairs ? tiles : max_pairs;
    kern<<<2 * pairs, kGemmThreads, PAIR_SMEM_BYTES, st>>>(ta, tb, tb2, p);
    return check_launch("xg_gemm_bias_act (CTA pairs)");
}

// Second pass of split-K: out = act(sum_s partial[s] + bias + residual), 4 columns per thread.
template <typename T>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const GemmParams p) {
    // Launched with programmatic stream serialisation: its CTAs may be placed while the GEMM is still draining; this
    // returns once the GEMM grid has completed and its partial sums are visible.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t n4 = (p.N + 3) / 4;
    const int64_t total = p.M * n4;
    const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (idx >= total) return;
    const int64_t row = idx / n4;
    const int64_t col0 = (idx - row * n4) * 4;
    const int ncol = (int)((p.N - col0) < 4 ? (p.N - col0) : 4);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const bool vec = (ncol == 4) && ((p.N & 3) == 0);
    const float* src = p.split.partial + row * p.N + col0;
    const int64_t plane = p.M * p.N;
    int s = 0;
    if (vec) {
        // four planes in flight per thread (a dependent chain of single loads costs about 0.3 us per split); the
        // additions stay in split order: deterministic
        for (; s + 4 <= p.splits; s += 4) {
            float4 f[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) f[j] = __ldcg(reinterpret_cast<const float4*>(src + (int64_t)(s + j) * plane));
#pragma unroll
            for (int j = 0; j < 4; ++j) { acc[0] += f[j].x; acc[1] += f[j].y; acc[2] += f[j].z; acc[3] += f[j].w; }
        }
        for (; s < p.splits; ++s) {
            const float4 f = __ldcg(reinterpret_cast<const float4*>(src + (int64_t)s * plane));
            acc[0] += f.x; acc[1] += f.y; acc[2] += f.z; acc[3] += f.w;
        }
    } else {
        for (; s < p.splits; ++s)
            for (int i = 0; i < ncol; ++i) acc[i] += src[(int64_t)s * plane + i];
    }
    const T* bias = reinterpret_cast<const T*>(p.bias);
    const T* resid = reinterpret_cast<const T*>(p.residual);
    T* out = reinterpret_cast<T*>(p.out);
    for (int i = 0; i < ncol; ++i) {
        float v = acc[i];
        if (bias) v += Cvt<T>::to_f(bias[col0 + i]);
        if (resid) v += Cvt<T>::to_f(resid[row * p.ldr + col0 + i]);
        out[row * p.ldc + col0 + i] = Cvt<T>::from_f(apply_act_out<T>(v, p.act));
    }
}

template <typename T, int BN, bool SWIGLU, bool B_MN>
int launch_gemm_tc(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const GemmParams& p,
                   cudaStream_t st) {
    using Cfg = GemmCfg<BN>;
    auto kern = gemm_tc_kernel<T, BN, SWIGLU, B_MN>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(XG_ERR_LAUNCH, "xg_gemm_bias_act: cannot reserve %d bytes of shared memory: %s", Cfg::SMEM_BYTES,
                    cudaGetErrorString(e));
    }
    const int64_t tiles = (int64_t)p.num_m_blocks * p.num_n_blocks * p.splits * batch_of(p);
    const int grid = (int)(tiles < num_sms() ? tiles : num_sms());
    kern<<<grid, kGemmThreads, Cfg::SMEM_BYTES, st>>>(ta, tb, tb2, p);
    int rc = check_launch("xg_gemm_bias_act");
    if (rc != XG_OK || p.splits <= 1) return rc;
    const int64_t total = p.M * ((p.N + 3) / 4);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((total + 255) / 256));
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;  // overlap this launch's latency with the GEMM's tail
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaError_t le = cudaLaunchKernelEx(&cfg, splitk_reduce_kernel<T>, p);
    if (le != cudaSuccess) {
        cudaGetLastError();
        return fail(XG_ERR_LAUNCH, "xg_gemm_bias_act (split-K reduce): %s", cudaGetErrorString(le));
    }
    return XG_OK;
}


// ---------------------------------------------------------------------------------------------------------
// Grouped dense layers: `count` problems of one shape whose operands live wherever the caller has them
// (a pointer per entry, no stacked copy). The persistent single-CTA kernel above, with the entry's tensor maps and
// pointers taken from a table in the kernel's parameter space instead of a third tensor-map coordinate.
// ---------------------------------------------------------------------------------------------------------
constexpr int kGroupMax = 12;  // entries per launch: 12 x (2 tensor maps + 3 pointers) = 3360 bytes of parameters
struct GroupTable {
    CUtensorMap a[kGroupMax];
    CUtensorMap w[kGroupMax];
    void* out[kGroupMax];
    const void* bias[kGroupMax];
    const void* resid[kGroupMax];
};

template <typename T, int BN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_group_kernel(const __grid_constant__ GroupTable tab, const GemmParams p, const int count) {
    using Cfg = GemmCfg<BN>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * Cfg::A_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
    uint64_t* full_bar = bars;
    uint64_t* empty_bar = bars + STAGES;
    uint64_t* tmem_full = bars + 2 * STAGES;
    uint64_t* tmem_empty = bars + 2 * STAGES + 2;
    uint64_t* drain_bar = bars + 2 * STAGES + 4;
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 5);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(&tmem_full[a], 1);
            ptx::mbar_init(&tmem_empty[a], 4);
        }
        ptx::mbar_init(drain_bar, 1);
        *abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::fence_proxy_async();
    }
    if (warp == 1) ptx::tmem_alloc(tmem_base_slot, Cfg::TMEM_COLS);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    const int tiles_per_entry = p.num_m_blocks * p.num_n_blocks;
    const int num_tiles = tiles_per_entry * count;  // work units: (entry, tile)
    const int nkb = p.num_k_blocks;

    if (warp == 0) {
        if (ptx::elect_one()) {
            int stage = 0;
            uint32_t phase = 0, armed = 0, armed_phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const int entry = t / tiles_per_entry;
                int mb, nb;
                tile_coords(t - entry * tiles_per_entry, p.num_m_blocks, p.num_n_blocks, mb, nb);
                const CUtensorMap* ta = &tab.a[entry];
                const CUtensorMap* tw = &tab.w[entry];
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!ptx::mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
                    ptx::mbar_arrive_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
                    ptx::tma_load_2d(smem_a + stage * Cfg::A_BYTES, ta, &full_bar[stage], kb * BK, mb * BM);
                    if (B_MN) {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            ptx::tma_load_2d(smem_b + stage * Cfg::B_BYTES + j * (BK * 128), tw, &full_bar[stage], nb * BN + j * 64, kb * BK);
                    } else {
                        ptx::tma_load_2d(smem_b + stage * Cfg::B_BYTES, tw, &full_bar[stage], kb * BK, nb * BN);
                    }
                    armed |= 1u << stage;
                    armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                atomicOr(&g_tc_status[0], 1u);
                for (int s = 0; s < STAGES; ++s) {
                    if (armed & (1u << s)) {
                        const uint64_t t0 = ptx::globaltimer_ns();
                        while (!ptx::mbar_try_wait(&full_bar[s], (armed_phase >> s) & 1u)) {
                            if (ptx::globaltimer_ns() - t0 > ptx::kWaitLimitNs) break;
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (ptx::elect_one()) {
            constexpr uint32_t idesc = ptx::make_idesc_f16(std::is_same<T, __nv_bfloat16>::value ? 1 : 0, BM, BN, B_MN ? 1 : 0);
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                if (!ptx::mbar_wait_bounded(&tmem_empty[acc], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                ptx::tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!ptx::mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
                    ptx::tc_fence_after();
                    const uint32_t a_addr = ptx::smem_u32(smem_a + stage * Cfg::A_BYTES);
                    const uint32_t b_addr = ptx::smem_u32(smem_b + stage * Cfg::B_BYTES);
                    const uint64_t da = ptx::make_kmajor_sw128_desc(a_addr);
                    const uint64_t db = B_MN ? ptx::make_mnmajor_sw128_desc(b_addr, BK * 128) : ptx::make_kmajor_sw128_desc(b_addr);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        ptx::mma_f16_ss(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(B_MN ? k * 128 : k * 2), idesc, (kb | k) != 0 ? 1u : 0u);
                    ptx::tc_commit(&empty_bar[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                ptx::tc_commit(&tmem_full[acc]);
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
            if (!ok) {
                atomicOr(&g_tc_status[0], 2u);
                ptx::tc_commit(drain_bar);
                const uint64_t t0 = ptx::globaltimer_ns();
                while (!ptx::mbar_try_wait(drain_bar, 0)) {
                    if (ptx::globaltimer_ns() - t0 > ptx::kWaitLimitNs) break;
                }
            }
        }
    } else {
        const int quad = warp & 3;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            const int entry = t / tiles_per_entry;
            int mb, nb;
            tile_coords(t - entry * tiles_per_entry, p.num_m_blocks, p.num_n_blocks, mb, nb);
            if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(&tmem_full[acc], acc_phase, abort_flag))) { ok = false; break; }
            ptx::tc_fence_after();
            GemmParams pe = p;  // this entry's pointers; everything else is shared by the group
            pe.out = tab.out[entry];
            pe.bias = tab.bias[entry];
            pe.residual = tab.resid[entry];
            const int64_t row = (int64_t)mb * BM + quad * 32 + lane;
            epilogue_tile<T, BN, false>(pe, tmem_base, acc, quad, row, row < p.M, nb, 0, 0);
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&tmem_empty[acc]);
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
        if (!ok && lane == 0) atomicOr(&g_tc_status[0], 4u);
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

template <typename T, int BN, bool B_MN>
int launch_gemm_group(const GroupTable& tab, const GemmParams& p, int count, cudaStream_t st) {
    using Cfg = GemmCfg<BN>;
    auto kern = gemm_tc_group_kernel<T, BN, B_MN>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(XG_ERR_LAUNCH, "xg_gemm_group_bias_act: cannot reserve %d bytes of shared memory: %s", Cfg::SMEM_BYTES,
                    cudaGetErrorString(e));
    }
    const int64_t tiles = (int64_t)p.num_m_blocks * p.num_n_blocks * count;
    const int grid = (int)(tiles < num_sms() ? tiles : num_sms());
    kern<<<grid, kGemmThreads, Cfg::SMEM_BYTES, st>>>(tab, p, count);
    return check_launch("xg_gemm_group_bias_act");
}

template <typename T>
int gemm_group_dispatch(const void* const* A, const void* const* W, const void* const* bias, const void* const* residual,
                        void* const* out, int64_t count, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldc,
                        int64_t ldr, int trans_b, int act, cudaStream_t st) {
    constexpr bool is_bf16 = std::is_same<T, __nv_bfloat16>::value;
    const int64_t mblk = (M + BM - 1) / BM;
    int bn = 256;
    if (count * mblk * ((N + 255) / 256) < num_sms()) bn = 128;
    if (bn == 128 && count * mblk * ((N + 127) / 128) < num_sms()) bn = 64;
    GemmParams p;
    p.out = nullptr;
    p.bias = nullptr;
    p.residual = nullptr;
    p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldr = ldr;
    p.act = act;
    p.mode = kModePlain;
    p.split.partial = nullptr;
    p.num_m_blocks = (int)mblk;
    p.num_n_blocks = (int)((N + bn - 1) / bn);
    p.num_k_blocks = (int)((K + BK - 1) / BK);
    p.splits = 1;
    for (int64_t first = 0; first < count; first += kGroupMax) {
        const int n = (int)((count - first) < kGroupMax ? (count - first) : kGroupMax);
        GroupTable tab;
        bool vec = (ldc % 8 == 0), bias_vec = true;
        for (int e = 0; e < n; ++e) {
            const void* a = A[first + e];
            const void* w = W[first + e];
            void* o = out[first + e];
            if (!a || !w || !o) return fail(XG_ERR_INVALID_ARG, "xg_gemm_group_bias_act: null pointer in entry %lld", (long long)(first + e));
            if (!aligned16(a) || !aligned16(w))
                return fail(XG_ERR_UNSUPPORTED, "xg_gemm_group_bias_act: entry %lld: A/W must be 16-byte aligned", (long long)(first + e));
            const bool w_ok = trans_b ? make_tmap_2d_16bit(&tab.w[e], w, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, (uint32_t)bn, BK, is_bf16)
                                      : make_tmap_2d_16bit(&tab.w[e], w, (uint64_t)K, (uint64_t)N, (uint64_t)ldw, BK, 64, is_bf16);
            if (!w_ok || !make_tmap_2d_16bit(&tab.a[e], a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM, BK, is_bf16))
                return fail(XG_ERR_UNSUPPORTED, "xg_gemm_group_bias_act: tensor-map encoding failed for entry %lld", (long long)(first + e));
            tab.out[e] = o;
            tab.bias[e] = bias ? bias[first + e] : nullptr;
            tab.resid[e] = residual ? residual[first + e] : nullptr;
            vec = vec && aligned16(o) && (!tab.resid[e] || (ldr % 8 == 0 && aligned16(tab.resid[e])));
            bias_vec = bias_vec && (!tab.bias[e] || aligned16(tab.bias[e]));
        }
        for (int e = n; e < kGroupMax; ++e) {  // unused slots: valid descriptors, never dereferenced
            tab.a[e] = tab.a[0];
            tab.w[e] = tab.w[0];
            tab.out[e] = nullptr;
            tab.bias[e] = nullptr;
            tab.resid[e] = nullptr;
        }
        p.vec_ok = vec ? 1 : 0;
        p.bias_vec_ok = bias_vec ? 1 : 0;
        int rc;
        if (!trans_b) {
            rc = bn == 256 ? launch_gemm_group<T, 256, true>(tab, p, n, st)
                           : (bn == 128 ? launch_gemm_group<T, 128, true>(tab, p, n, st) : launch_gemm_group<T, 64, true>(tab, p, n, st));
        } else {
            rc = bn == 256 ? launch_gemm_group<T, 256, false>(tab, p, n, st)
                           : (bn == 128 ? launch_gemm_group<T, 128, false>(tab, p, n, st) : launch_gemm_group<T, 64, false>(tab, p, n, st));
        }
        if (rc != XG_OK) return rc;
    }
    return XG_OK;
}

}  // namespace

// CTA pairs pay off once there are enough 256-row tiles to keep every pair busy. XG_GEMM_PAIRS=0/1 overrides.
bool use_cta_pairs(int64_t M, int64_t N, int out_bn) {
    static const int forced = []() {
        const char* e = getenv("XG_GEMM_PAIRS");
        return e ? (e[0] == '0' ? 0 : 1) : -1;
    }();
    if (forced >= 0) return forced == 1;
    const int64_t tiles = ((M + 255) / 256) * ((N + out_bn - 1) / out_bn);
    return tiles >= num_sms() / 2;  // measured on B200: +10 % (plain) / +8 % (SwiGLU) at 8192 x 4096 x 11008
}

// Tile width and split-K factor for an [M, N, K] problem given `ws_bytes` of fp32 scratch (0 = none).
// Larger M: the widest tile that still gives every SM work, no split. M <= 128 is the weight-streaming regime, where
// what a CTA takes in through its SM decides: (128 + bn) rows of 128 bytes per k-block, and the activations again
// for every column tile. There the plan is the cheapest of every (tile width, split) that runs as a single wave, by a
// cost model in microseconds fitted to sweeps on B200 (K = 4096; M = 16..128; N = 512..11008; tile widths 64 / 128 /
// 256; 1..16 splits; CUDA-graph replay):
//   ingest  : 8.5 us per MB a CTA takes in (about 118 KB/us per SM), times the waves;
//   tile    : 0.01 us per tile column (the epilogue of a wide tile is served by the same four warps);
//   launch  : 2.5 us;
//   a split : 4 us more (second launch, drain) and the fp32 partial sums written and read back: 0.13 us per MB while
//             weights + partial sums stay within L2, 0.67 us per MB beyond that.
// Measured examples (us; this plan / the previous one, which knew only 256-wide split tiles and took the narrowest
// tile unsplit): 128 x 4096 x 4096 13.0 / 15.3; 64 x 4096 x 4096 11.1 / 14.2; 128 x 4096 x 2048 10.8 / 16.1;
// 128 x 4096 x 11008 21.3 / 27.2; 64 x 4096 x 11008 19.9 / 27.0. At M = 256 a split through scratch loses to the
// unsplit kernel (15.6 us vs 22.4 / 19.8 / 29.8 us for 2 / 4 / 8 splits at N = K = 4096); those shapes belong to the
// cluster kernel, which reduces through shared memory.
GemmPlan plan_gemm(int64_t M, int64_t N, int64_t K, int64_t ws_bytes, int sms) {
    GemmPlan pl;
    const int64_t mblk = (M + BM - 1) / BM;
    pl.bn = 256;
    if (mblk * ((N + 255) / 256) < sms) pl.bn = 128;
    if (pl.bn == 128 && mblk * ((N + 127) / 128) < sms) pl.bn = 64;
    pl.splits = 1;
    const int64_t nkb = (K + BK - 1) / BK;
    if (M > 128 || nkb < 8) return pl;
    const double w_mb = 2.0 * (double)N * (double)K / 1e6;
    double best = 1e30;
    for (int bn = 64; bn <= 256; bn *= 2) {
        const int64_t tiles = mblk * ((N + bn - 1) / bn);
        const double per_kblock_mb = (double)(BM + bn) * 128.0 / 1e6;
        for (int s = 1; s <= 16; ++s) {
            if (s > 1 && (s * 4 > nkb || (int64_t)s * M * N * 4 > ws_bytes || tiles * s > sms)) break;
            const double waves = (double)((tiles * s + sms - 1) / sms);
            double c = waves * (double)((nkb + s - 1) / s) * per_kblock_mb * 8.5 + 0.01 * bn + 2.5;
            if (s > 1) {
                const double partial_mb = 2.0 * s * (double)M * (double)N * 4.0 / 1e6;
                c += 4.0 + partial_mb * (w_mb + partial_mb < 96.0 ? 0.13 : 0.67);
            }
            if (c < best) {
                best = c;
                pl.bn = bn;
                pl.splits = s;
            }
        }
    }
    return pl;
}

int64_t gemm_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    int S = 0, tn = 0;
    if (plan_ksplit(M, N, K, XG_BF16, &S, &tn)) return 0;  // the cluster kernel reduces through shared memory
    const GemmPlan pl = plan_gemm(M, N, K, (int64_t)1 << 40, num_sms());
    return pl.splits > 1 ? (int64_t)pl.splits * M * N * 4 : 0;
}

namespace {

template <typename T>
int gemm_tc_dispatch(const void* A, const void* B, const void* bias, const void* residual, void* out, int64_t M,
                     int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr, int trans_b, int act,
                     void* workspace, int64_t ws_bytes, bool force_split, const GemmExtras* ex, cudaStream_t st) {
    constexpr bool is_bf16 = std::is_same<T, __nv_bfloat16>::value;
    if (ex && ex->rope_cos) ws_bytes = 0;  // the rotary epilogue lives in the GEMM kernel: no split-K
    const int64_t mblk = (M + BM - 1) / BM;
    if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) ws_bytes = 0;
    GemmPlan pl = plan_gemm(M, N, K, ws_bytes, num_sms());
    if (force_split && pl.splits == 1 && ws_bytes >= 2 * M * N * 4 && (K + BK - 1) / BK >= 2) {
        pl.bn = 256;  // the caller asked for the split path: the smallest split that the scratch holds
        pl.splits = 2;
    }
    if (ex && ex->rope_cos && pl.bn < 128) pl.bn = 128;  // a head (<= 128 columns) must not straddle two tiles
    const int bn = pl.bn;

    CUtensorMap ta, tb;
    const bool b_ok = trans_b ? make_tmap_2d_16bit(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint32_t)bn, BK, is_bf16)
                              : make_tmap_2d_16bit(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, 64, is_bf16);
    if (!make_tmap_2d_16bit(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM, BK, is_bf16) || !b_ok)
        return fail(XG_ERR_UNSUPPORTED, "xg_gemm_bias_act: tensor-map encoding failed (M=%lld N=%lld K=%lld lda=%lld ldb=%lld)",
                    (long long)M, (long long)N, (long long)K, (long long)lda, (long long)ldb);
    GemmParams p;
    p.out = out;
    p.bias = bias;
    p.residual = residual;
    p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldr = ldr;
    p.act = act;
    p.mode = kModePlain;
    p.split.partial = nullptr;
    if (ex && ex->rope_cos) {
        p.mode = kModeRope;
        p.rope.cos = ex->rope_cos;
        p.rope.sin = ex->rope_sin;
        p.rope.S = ex->rope_S;
        p.rope.D = ex->rope_D;
    }
    p.vec_ok = (ldc % 8 == 0) && aligned16(out) && (!residual || (ldr % 8 == 0 && aligned16(residual)));
    p.bias_vec_ok = bias ? aligned16(bias) : 0;
    if (trans_b && pl.splits == 1 && use_cta_pairs(M, N, 256)) {
        // large problem: 256 x 256 tiles on CTA pairs (W box = 128 rows per CTA)
        CUtensorMap tbp;
        if (!make_tmap_2d_16bit(&tbp, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 128, BK, is_bf16))
            return fail(XG_ERR_UNSUPPORTED, "xg_gemm_bias_act: tensor-map encoding failed");
        p.num_m_blocks = (int)((M + 255) / 256);
        p.num_n_blocks = (int)((N + 255) / 256);
        p.num_k_blocks = (int)((K + BK - 1) / BK);
        p.splits = 1;
        return launch_gemm_pair<T, false>(ta, tbp, tbp, p, st);
    }
    p.num_m_blocks = (int)mblk;
    p.num_n_blocks = (int)((N + bn - 1) / bn);
    p.num_k_blocks = (int)((K + BK - 1) / BK);
    p.splits = pl.splits;
    if (pl.splits > 1) p.split.partial = reinterpret_cast<float*>(workspace);  // (never together with the rotary epilogue)
    if (!trans_b) {
        switch (bn) {
            case 256: return launch_gemm_tc<T, 256, false, true>(ta, tb, tb, p, st);
            case 128: return launch_gemm_tc<T, 128, false, true>(ta, tb, tb, p, st);
            default: return launch_gemm_tc<T, 64, false, true>(ta, tb, tb, p, st);
        }
    }
    switch (bn) {
        case 256: return launch_gemm_tc<T, 256, false, false>(ta, tb, tb, p, st);
        case 128: return launch_gemm_tc<T, 128, false, false>(ta, tb, tb, p, st);
        default: return launch_gemm_tc<T, 64, false, false>(ta, tb, tb, p, st);
    }
}

template <typename T>
int gemm_swiglu_dispatch(const void* A, const void* Wg, const void* Wu, void* out, int64_t M, int64_t N, int64_t K,
                         int64_t lda, int64_t ldw, int64_t ldc, cudaStream_t st) {
    constexpr bool is_bf16 = std::is_same<T, __nv_bfloat16>::value;
    CUtensorMap ta, tg, tu;
    if (!make_tmap_2d_16bit(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM, BK, is_bf16) ||
        !make_tmap_2d_16bit(&tg, Wg, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, 128, BK, is_bf16) ||
        !make_tmap_2d_16bit(&tu, Wu, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, 128, BK, is_bf16))
        return fail(XG_ERR_UNSUPPORTED, "xg_gemm_swiglu: tensor-map encoding failed");
    GemmParams p;
    p.out = out;
    p.bias = nullptr;
    p.residual = nullptr;
    p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldr = 0;
    p.act = XG_ACT_NONE;
    p.mode = kModePlain;
    p.vec_ok = (ldc % 8 == 0) && aligned16(out);
    p.bias_vec_ok = 0;
    p.num_n_blocks = (int)((N + 127) / 128);
    p.num_k_blocks = (int)((K + BK - 1) / BK);
    p.splits = 1;
    p.split.partial = nullptr;
    if (use_cta_pairs(M, N, 128)) {
        p.num_m_blocks = (int)((M + 255) / 256);
        return launch_gemm_pair<T, true>(ta, tg, tu, p, st);
    }
    p.num_m_blocks = (int)((M + BM - 1) / BM);
    return launch_gemm_tc<T, 256, true, false>(ta, tg, tu, p, st);
}

}  // namespace

// Entry used by xg_gemm_bias_act for 16-bit dtypes; W is [N, K] (trans_b = 1) or [K, N] (trans_b = 0).
int gemm_tc_entry(const void* A, const void* B, const void* bias, const void* residual, void* out, int64_t M, int64_t N,
                  int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr, int trans_b, int act, int dtype,
                  void* workspace, int64_t ws_bytes, cudaStream_t st, bool force_split, const GemmExtras* extras) {
    if (!aligned16(A) || !aligned16(B) || lda % 8 != 0 || ldb % 8 != 0)
        return fail(XG_ERR_UNSUPPORTED, "xg_gemm_bias_act: A/W must be 16-byte aligned with row strides multiple of 8 elements");
    if (M * N == 0) return XG_OK;
    if (M > (int64_t)BM * 0x7fffff || N > (int64_t)64 * 0x7fffff || K > 0x7fffffff)
        return fail(XG_ERR_TOO_LARGE, "xg_gemm_bias_act: extent too large");
    if (trans_b && !force_split && !(extras && extras->rope_cos)) {
        // few output tiles: K split over the CTA pairs of a cluster, partial sums exchanged through shared memory
        int S = 0, tn = 0;
        if (plan_ksplit(M, N, K, dtype, &S, &tn))
            return gemm_tc_ksplit_entry(A, B, bias, residual, out, M, N, K, lda, ldb, ldc, ldr, act, dtype, S, tn, st);
    }
    if (dtype == XG_BF16)
        return gemm_tc_dispatch<__nv_bfloat16>(A, B, bias, residual, out, M, N, K, lda, ldb, ldc, ldr, trans_b, act, workspace, ws_bytes, force_split, extras, st);
    return gemm_tc_dispatch<__half>(A, B, bias, residual, out, M, N, K, lda, ldb, ldc, ldr, trans_b, act, workspace, ws_bytes, force_split, extras, st);
}

// ---- batched dense layers in one launch -----------------------------------------------------------------
// out[e] = act(A[e] @ W[e] + bias[e] + residual[e]) for e < batch, all entries of one shape: the persistent
// single-CTA kernel walks (entry, tile) units, its tensor maps carrying the batch as a third dimension.
// Returns XG_ERR_UNSUPPORTED (without a message for the caller to act on) when the strides do not fit a tensor map.
template <typename T>
static int bgemm_tc_dispatch(const void* A, const void* B, const void* bias, const void* residual, void* out, int64_t batch,
                             int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr,
                             int64_t sa, int64_t sb, int64_t sbias, int64_t sr, int64_t sc, int trans_b, int act,
                             cudaStream_t st) {
    constexpr bool is_bf16 = std::is_same<T, __nv_bfloat16>::value;
    const int64_t mblk = (M + BM - 1) / BM;
    int bn = 256;
    if (batch * mblk * ((N + 255) / 256) < num_sms()) bn = 128;
    if (bn == 128 && batch * mblk * ((N + 127) / 128) < num_sms()) bn = 64;
    CUtensorMap ta, tb;
    const bool b_ok = trans_b ? make_tmap_3d_16bit(&tb, B, (uint64_t)batch, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint64_t)sb, (uint32_t)bn, BK, is_bf16)
                              : make_tmap_3d_16bit(&tb, B, (uint64_t)batch, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, (uint64_t)sb, BK, 64, is_bf16);
    if (!b_ok || !make_tmap_3d_16bit(&ta, A, (uint64_t)batch, (uint64_t)M, (uint64_t)K, (uint64_t)lda, (uint64_t)sa, BM, BK, is_bf16))
        return fail(XG_ERR_UNSUPPORTED, "xg_bgemm_bias_act: tensor-map encoding failed");
    GemmParams p;
    p.out = out;
    p.bias = bias;
    p.residual = residual;
    p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldr = ldr;
    p.act = act;
    p.mode = kModePlain;
    p.vec_ok = (ldc % 8 == 0) && (sc % 8 == 0) && aligned16(out) && (!residual || (ldr % 8 == 0 && sr % 8 == 0 && aligned16(residual)));
    p.bias_vec_ok = bias ? (aligned16(bias) && sbias % 8 == 0) : 0;
    p.num_m_blocks = (int)mblk;
    p.num_n_blocks = (int)((N + bn - 1) / bn);
    p.num_k_blocks = (int)((K + BK - 1) / BK);
    p.splits = 1;
    p.mode = kModeBatch;
    p.batch.count = (int)batch;
    p.batch.bs_out = sc;
    p.batch.bs_bias = sbias;
    p.batch.bs_res = sr;
    if (!trans_b) {
        switch (bn) {
            case 256: return launch_gemm_tc<T, 256, false, true>(ta, tb, tb, p, st);
            case 128: return launch_gemm_tc<T, 128, false, true>(ta, tb, tb, p, st);
            default: return launch_gemm_tc<T, 64, false, true>(ta, tb, tb, p, st);
        }
    }
    switch (bn) {
        case 256: return launch_gemm_tc<T, 256, false, false>(ta, tb, tb, p, st);
        case 128: return launch_gemm_tc<T, 128, false, false>(ta, tb, tb, p, st);
        default: return launch_gemm_tc<T, 64, false, false>(ta, tb, tb, p, st);
    }
}

// True when the batched problem can run as one launch (16-bit dtype, TMA-addressable operands, more than one entry).
bool bgemm_single_launch_ok(const void* A, const void* B, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t lda,
                            int64_t ldb, int64_t sa, int64_t sb, int dtype) {
    if (dtype != XG_BF16 && dtype != XG_F16) return false;
    if (batch < 2 || batch > 65535 || M <= 0 || N <= 0 || K <= 0) return false;
    if (!aligned16(A) || !aligned16(B) || lda % 8 != 0 || ldb % 8 != 0) return false;
    if (sa <= 0 || sb <= 0 || sa % 8 != 0 || sb % 8 != 0) return false;  // a broadcast operand (stride 0) takes the per-entry path
    const int64_t units = batch * ((M + BM - 1) / BM) * ((N + 63) / 64);
    return units < 0x7fffffffLL && M <= (int64_t)BM * 0x7fffff && N <= (int64_t)64 * 0x7fffff && K <= 0x7fffffff;
}

int bgemm_tc_entry(const void* A, const void* B, const void* bias, const void* residual, void* out, int64_t batch, int64_t M,
                   int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr, int64_t sa, int64_t sb,
                   int64_t sbias, int64_t sr, int64_t sc, int trans_b, int act, int dtype, cudaStream_t st) {
    if (dtype == XG_BF16)
        return bgemm_tc_dispatch<__nv_bfloat16>(A, B, bias, residual, out, batch, M, N, K, lda, ldb, ldc, ldr, sa, sb, sbias, sr, sc, trans_b, act, st);
    return bgemm_tc_dispatch<__half>(A, B, bias, residual, out, batch, M, N, K, lda, ldb, ldc, ldr, sa, sb, sbias, sr, sc, trans_b, act, st);
}

// Grouped dense layers (one shape, a pointer per entry): see gemm_tc_group_kernel.
int gemm_group_entry(const void* const* A, const void* const* W, const void* const* bias, const void* const* residual,
                     void* const* out, int64_t count, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldc,
                     int64_t ldr, int trans_b, int act, int dtype, cudaStream_t st) {
    if (lda % 8 != 0 || ldw % 8 != 0)
        return fail(XG_ERR_UNSUPPORTED, "xg_gemm_group_bias_act: row strides must be multiples of 8 elements");
    if (M > (int64_t)BM * 0x7fffff || N > (int64_t)64 * 0x7fffff || K > 0x7fffffff ||
        count * ((M + BM - 1) / BM) * ((N + 63) / 64) > 0x7fffffffLL)
        return fail(XG_ERR_TOO_LARGE, "xg_gemm_group_bias_act: extent too large");
    if (dtype == XG_BF16)
        return gemm_group_dispatch<__nv_bfloat16>(A, W, bias, residual, out, count, M, N, K, lda, ldw, ldc, ldr, trans_b, act, st);
    return gemm_group_dispatch<__half>(A, W, bias, residual, out, count, M, N, K, lda, ldw, ldc, ldr, trans_b, act, st);
}

// ---- fp32 problems on the bf16 tensor cores ------------------------------------------------------------
// A3 [M, 3*Kp] and W3 [N, 3*Kp] hold the three bf16 planes of the fp32 operands (split_bf16x3.cu). The product is
// the sum of the six plane pairs whose weight is at least 2^-16, smallest first, accumulated in fp32 in TMEM by the
// ordinary bf16 kernels running over 6*Kp/64 k-blocks: about 2^-23 relative error per product, at one sixth of the
// bf16 rate. The epilogue adds the fp32 bias / residual, applies the activation and stores fp32 - or, for a layer
// that feeds another one, stores the result directly as that layer's three bf16 planes.
int gemm_f32x3_entry(const void* A3, const void* W3, const void* bias, const void* residual, void* out, int64_t M,
                     int64_t N, int64_t Kp, int64_t ldc, int64_t ldr, int act, int out_planes, cudaStream_t st) {
    if (M * N == 0) return XG_OK;
    if (Kp <= 0 || Kp % BK != 0) return fail(XG_ERR_INVALID_ARG, "xg_gemm_f32x3: the padded K must be a positive multiple of %d", BK);
    if (!aligned16(A3) || !aligned16(W3)) return fail(XG_ERR_UNSUPPORTED, "xg_gemm_f32x3: operands must be 16-byte aligned");
    if (out_planes && (!aligned16(out) || residual))
        return fail(XG_ERR_UNSUPPORTED, "xg_gemm_f32x3: the plane output must be 16-byte aligned and takes no residual");
    if (M > (int64_t)BM * 0x7fffff || N > (int64_t)64 * 0x7fffff || 6 * Kp > 0x7fffffff)
        return fail(XG_ERR_TOO_LARGE, "xg_gemm_f32x3: extent too large");
    GemmParams p;
    p.out = out;
    p.bias = bias;
    p.residual = residual;
    p.M = M; p.N = N; p.K = 3 * Kp; p.ldc = ldc; p.ldr = ldr;
    p.act = act;
    p.mode = kModePlain;
    // fp32 rows in 16-byte steps (four floats)
    p.vec_ok = (ldc % 4 == 0) && aligned16(out) && (!residual || (ldr % 4 == 0 && aligned16(residual)));
    p.bias_vec_ok = 0;
    p.splits = 1;
    p.mode = out_planes ? kModeF32Planes : kModeF32;
    p.f32.out_kp = out_planes ? (N + BK - 1) / BK * BK : 0;
    p.f32.seg_blocks = (int)(Kp / BK);
    p.f32.seg_a = 0x010120u;  // pairs (A plane, W plane): (0,2) (2,0) (1,1) (0,1) (1,0) (0,0)
    p.f32.seg_b = 0x001102u;
    p.f32.pad_ = 0;
    p.num_k_blocks = 6 * p.f32.seg_blocks;
    CUtensorMap ta, tb;
    if (!make_tmap_2d_16bit(&ta, A3, (uint64_t)M, (uint64_t)(3 * Kp), (uint64_t)(3 * Kp), BM, BK, true))
        return fail(XG_ERR_UNSUPPORTED, "xg_gemm_f32x3: tensor-map encoding failed");
    if (use_cta_pairs(M, N, 256)) {
        if (!make_tmap_2d_16bit(&tb, W3, (uint64_t)N, (uint64_t)(3 * Kp), (uint64_t)(3 * Kp), 128, BK, true))
            return fail(XG_ERR_UNSUPPORTED, "xg_gemm_f32x3: tensor-map encoding failed");
        p.num_m_blocks = (int)((M + 255) / 256);
        p.num_n_blocks = (int)((N + 255) / 256);
        return launch_gemm_pair<__nv_bfloat16, false>(ta, tb, tb, p, st);
    }
    const GemmPlan pl = plan_gemm(M, N, 6 * Kp, 0, num_sms());
    if (!make_tmap_2d_16bit(&tb, W3, (uint64_t)N, (uint64_t)(3 * Kp), (uint64_t)(3 * Kp), (uint32_t)pl.bn, BK, true))
        return fail(XG_ERR_UNSUPPORTED, "xg_gemm_f32x3: tensor-map encoding failed");
    p.num_m_blocks = (int)((M + BM - 1) / BM);
    p.num_n_blocks = (int)((N + pl.bn - 1) / pl.bn);
    switch (pl.bn) {
        case 256: return launch_gemm_tc<__nv_bfloat16, 256, false, false>(ta, tb, tb, p, st);
        case 128: return launch_gemm_tc<__nv_bfloat16, 128, false, false>(ta, tb, tb, p, st);
        default: return launch_gemm_tc<__nv_bfloat16, 64, false, false>(ta, tb, tb, p, st);
    }
}

// ---- split-K on a fixed, library-owned scratch array (nothing is allocated by anyone) ------------------
constexpr int64_t kStaticScratchBytes = 32ll << 20;  // 32 MiB, held by every GPU that loads the library
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

int64_t static_scratch_capacity() { return kStaticScratchBytes; }

// Device address of the scratch array on the current device. In host code the array's name is only a
// handle for the runtime, not a pointer a kernel could use, so the address is resolved with
// cudaGetSymbolAddress - once per device, with that device current - and cached.
static int static_scratch_address(void** out) {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static void* cached[kMaxDevices] = {nullptr};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        return fail(XG_ERR_DEVICE, "xg_gemm_bias_act_static: no usable current device");
    }
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == nullptr) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            cudaGetLastError();
            return fail(XG_ERR_DEVICE, "xg_gemm_bias_act_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        }
        cached[dev] = ptr;
    }
    *out = cached[dev];
    return XG_OK;
}

int gemm_tc_static_entry(const void* A, const void* B, const void* bias, const void* residual, void* out, int64_t M,
                         int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr, int trans_b, int act,
                         int dtype, cudaStream_t st) {
    if (M < 0 || N < 0 || K < 0) return fail(XG_ERR_INVALID_ARG, "xg_gemm_bias_act_static: negative extent");
    if (M == 0 || N == 0) return XG_OK;
    // the extents are bounded before any product of them is formed: M * N of huge extents could wrap
    if (M > kStaticScratchBytes || N > kStaticScratchBytes)
        return fail(XG_ERR_TOO_LARGE, "xg_gemm_bias_act_static: M = %lld, N = %lld is beyond the built-in scratch array; use "
                    "xg_gemm_bias_act_ws with your own workspace", (long long)M, (long long)N);
    const int64_t need = 2 * M * N * 4;  // two fp32 partial-sum planes is the least a split needs
    if (need > kStaticScratchBytes)
        return fail(XG_ERR_TOO_LARGE,
                    "xg_gemm_bias_act_static: M*N = %lld needs %lld bytes of scratch for a 2-way split, the built-in array "
                    "holds %lld; use xg_gemm_bias_act_ws with your own workspace",
                    (long long)(M * N), (long long)need, (long long)kStaticScratchBytes);
    if ((K + BK - 1) / BK < 2)
        return fail(XG_ERR_UNSUPPORTED, "xg_gemm_bias_act_static: K = %lld is a single k-block, nothing to split", (long long)K);
    void* scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc != XG_OK) return rc;
    return gemm_tc_entry(A, B, bias, residual, out, M, N, K, lda, ldb, ldc, ldr, trans_b, act, dtype, scratch,
                         kStaticScratchBytes, st, /*force_split=*/true);
}

int gemm_rope_entry(const void* A, const void* W, const void* cos, const void* sin, void* out, int64_t M, int64_t N, int64_t K,
                    int64_t lda, int64_t ldw, int64_t ldc, int64_t S, int64_t D, int dtype, cudaStream_t st) {
    if (D != 64 && D != 128) return fail(XG_ERR_UNSUPPORTED, "xg_gemm_rope: head_dim must be 64 or 128");
    if (N % D != 0 || S <= 0) return fail(XG_ERR_INVALID_ARG, "xg_gemm_rope: N must be a multiple of head_dim and S positive");
    if (!aligned16(cos) || !aligned16(sin) || !aligned16(out) || ldc % 8 != 0)
        return fail(XG_ERR_UNSUPPORTED, "xg_gemm_rope: tables and output rows must be 16-byte addressable");
    GemmExtras ex;
    ex.rope_cos = cos;
    ex.rope_sin = sin;
    ex.rope_S = S;
    ex.rope_D = (int)D;
    return gemm_tc_entry(A, W, nullptr, nullptr, out, M, N, K, lda, ldw, ldc, 0, 1, XG_ACT_NONE, dtype, nullptr, 0, st, false, &ex);
}

int gemm_swiglu_entry(const void* A, const void* Wg, const void* Wu, void* out, int64_t M, int64_t N, int64_t K,
                      int64_t lda, int64_t ldw, int64_t ldc, int dtype, cudaStream_t st) {
    if (!aligned16(A) || !aligned16(Wg) || !aligned16(Wu) || lda % 8 != 0 || ldw % 8 != 0)
        return fail(XG_ERR_UNSUPPORTED, "xg_gemm_swiglu: A/W must be 16-byte aligned with row strides multiple of 8 elements");
    if (M * N == 0) return XG_OK;
    if (M > (int64_t)BM * 0x7fffff || N > (int64_t)64 * 0x7fffff || K > 0x7fffffff)
        return fail(XG_ERR_TOO_LARGE, "xg_gemm_swiglu: extent too large");
    if (dtype == XG_BF16) return gemm_swiglu_dispatch<__nv_bfloat16>(A, Wg, Wu, out, M, N, K, lda, ldw, ldc, st);
    return gemm_swiglu_dispatch<__half>(A, Wg, Wu, out, M, N, K, lda, ldw, ldc, st);
}

int read_tc_status(unsigned int* host_out, int reset) {
    unsigned int v[4] = {0, 0, 0, 0};
    if (cudaMemcpyFromSymbol(v, g_tc_status, sizeof(v)) != cudaSuccess) {
        cudaGetLastError();
        return fail(XG_ERR_DEVICE, "xg_tc_status: cannot read device status");
    }
    *host_out = v[0];
    if (reset && v[0] != 0) {
        unsigned int z[4] = {0, 0, 0, 0};
        cudaMemcpyToSymbol(g_tc_status, z, sizeof(z));
    }
    return XG_OK;
}

}  // namespace xg
