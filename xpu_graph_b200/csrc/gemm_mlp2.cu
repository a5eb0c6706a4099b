// Two chained dense layers in one kernel: out = act2(act1(x W1^T + b1) W2^T + b2) for narrow 16-bit layers
// (N1, N2 <= 256), the place of the reference's serial-matmul kernels (targets/mlu/fuse_densetower.py:272-316,
// triton_kernel/fused_serial_mm_2dot.py:142): the hidden activation never leaves the SM.
//
// One persistent CTA per SM walks 128-row blocks of x. Per block:
//   phase 1  acc1[128 x N1] = x_blk W1^T   tcgen05.mma, both operands streamed by TMA through a 3-stage ring
//   hand-over the eight epilogue warps read acc1 from TMEM, add b1, apply act1, round to the 16-bit type (the rounding
//            the unfused graph does when it stores the hidden tensor) and write the result into shared memory in the
//            K-major 128-byte-swizzled layout an MMA A operand wants (the layout TMA would have produced)
//   phase 2  acc2[128 x N2] = h W2^T        A = the hidden block in shared memory, W2 streamed through the same ring
//   epilogue acc2 + b2, act2 -> out
// acc1 and acc2 live in different TMEM columns, so phase 1 of the next block runs while the epilogue of the current
// one drains acc2. Ragged extents need no special code: TMA zero-fills outside the tensors, hidden columns beyond N1
// are written as zeros, rows beyond M are not stored.
#include "common.cuh"
#include "sm100_ptx.cuh"

#include <type_traits>

namespace xg {

// Status word of this kernel (device globals are per translation unit without -rdc).
__device__ unsigned int g_mlp_status[4];

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int MAX_N = 256;
constexpr int STAGES = 3;
constexpr int A_BYTES = BM * BK * 2;        // 16 KiB: a [128 x 64] block of x
constexpr int B_BYTES = MAX_N * BK * 2;     // 32 KiB: up to 256 weight rows x 64 columns
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int H_SLABS = MAX_N / BK;         // the hidden block as 64-column slabs of [128 rows x 128 bytes]
constexpr int H_BYTES = H_SLABS * A_BYTES;  // 64 KiB
constexpr int MLP_SMEM_BYTES = STAGES * STAGE_BYTES + H_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int EPI_WARPS = 8;                // two per TMEM lane quadrant: a single warp per scheduler is latency-bound
constexpr int MLP_THREADS = 64 + EPI_WARPS * 32;  // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue
constexpr int TMEM_COLS = 512;              // acc1 [0, 256), acc2 [256, 512)

struct MlpParams {
    void* out;
    const void* b1;
    const void* b2;
    int64_t M, ldc;
    int N1, N2;          // layer widths
    int n1p, n2p;        // MMA N of the two phases: the widths rounded up to 16
    int nk1, nk2;        // 64-column k-blocks of phase 1 (over K1) and phase 2 (over N1)
    int num_m_blocks;
    int act1, act2;
    int out_vec_ok;      // out and ldc allow 16-byte stores
    int b1_vec_ok, b2_vec_ok;
};
static_assert(sizeof(MlpParams) <= 128, "three tensor maps and this struct stay within a 512-byte parameter block");

__device__ __forceinline__ float apply_act(float v, int act) {
    switch (act) {
        case XG_ACT_GELU: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
        case XG_ACT_RELU: return v > 0.f ? v : 0.f;
        case XG_ACT_SILU: return __fdividef(v, 1.0f + __expf(-v));
        case XG_ACT_SIGMOID: return __fdividef(1.0f, 1.0f + __expf(-v));
        default: return v;
    }
}

// 32 accumulator columns [col0, col0 + 32) of this thread's row: + bias (columns < n only), activation.
template <typename T>
__device__ __forceinline__ void finish_chunk(float (&v)[32], const T* bias, bool bias_vec_ok, int col0, int n, int act) {
    const bool full = col0 + 32 <= n;
    if (bias != nullptr) {
        if (full && bias_vec_ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
                const Vec16<T> bv = ld16(bias + col0 + i);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[i + j] += Cvt<T>::to_f(bv.v[j]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (col0 + i < n) v[i] += Cvt<T>::to_f(bias[col0 + i]);
        }
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = apply_act(v[i], act);
}

template <typename T>
__global__ void __launch_bounds__(MLP_THREADS, 1)
mlp2_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w1,
            const __grid_constant__ CUtensorMap tmap_w2, const MlpParams p) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: required by the 128-byte swizzle pattern shared by TMA and the MMA descriptors.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;                           // [STAGES][A_BYTES]
    uint8_t* smem_b = smem + STAGES * A_BYTES;        // [STAGES][B_BYTES]
    uint8_t* smem_h = smem + STAGES * STAGE_BYTES;    // [H_SLABS][A_BYTES]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_h + H_BYTES);
    uint64_t* full_bar = bars;                // [STAGES]
    uint64_t* empty_bar = bars + STAGES;      // [STAGES]
    uint64_t* acc1_full = bars + 2 * STAGES;  // phase 1 of a block has completed
    uint64_t* h_full = acc1_full + 1;         // the hidden block is in shared memory (every epilogue thread arrives)
    uint64_t* acc2_full = acc1_full + 2;      // phase 2 of a block has completed
    uint64_t* acc2_empty = acc1_full + 3;     // the epilogue warps have read acc2 (one arrival per warp)
    uint64_t* drain_bar = acc1_full + 4;
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc1_full + 5);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        ptx::mbar_init(acc1_full, 1);
        ptx::mbar_init(h_full, EPI_WARPS * 32);
        ptx::mbar_init(acc2_full, 1);
        ptx::mbar_init(acc2_empty, EPI_WARPS);
        ptx::mbar_init(drain_bar, 1);
        *abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::fence_proxy_async();
    }
    if (warp == 1) ptx::tmem_alloc(tmem_base_slot, TMEM_COLS);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    const uint32_t w1_bytes = (uint32_t)p.n1p * BK * 2, w2_bytes = (uint32_t)p.n2p * BK * 2;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (ptx::elect_one()) {
            ptx::prefetch_tensormap(&tmap_x);
            ptx::prefetch_tensormap(&tmap_w1);
            ptx::prefetch_tensormap(&tmap_w2);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t armed = 0, armed_phase = 0;  // stages with a load of this thread in flight, and the parity of each
            bool ok = true;
            for (int mb = blockIdx.x; mb < p.num_m_blocks && ok; mb += gridDim.x) {
                for (int kb = 0; kb < p.nk1 + p.nk2; ++kb) {
                    if (!ptx::mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
                    if (kb < p.nk1) {
                        ptx::mbar_arrive_expect_tx(&full_bar[stage], A_BYTES + w1_bytes);
                        ptx::tma_load_2d(smem_a + stage * A_BYTES, &tmap_x, &full_bar[stage], kb * BK, mb * BM);
                        ptx::tma_load_2d(smem_b + stage * B_BYTES, &tmap_w1, &full_bar[stage], kb * BK, 0);
                    } else {
                        ptx::mbar_arrive_expect_tx(&full_bar[stage], w2_bytes);
                        ptx::tma_load_2d(smem_b + stage * B_BYTES, &tmap_w2, &full_bar[stage], (kb - p.nk1) * BK, 0);
                    }
                    armed |= 1u << stage;
                    armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                // Unwinding: let this thread's own copies land before the CTA gives up its shared memory.
                atomicOr(&g_mlp_status[0], 1u);
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
            constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
            const uint32_t idesc1 = ptx::make_idesc_f16(fmt, BM, p.n1p, 0);
            const uint32_t idesc2 = ptx::make_idesc_f16(fmt, BM, p.n2p, 0);
            const uint32_t h_addr = ptx::smem_u32(smem_h);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t blk = 0;  // blocks done so far: parity of the per-block barriers
            bool ok = true;
            for (int mb = blockIdx.x; mb < p.num_m_blocks && ok; mb += gridDim.x, ++blk) {
                // phase 1 (acc1 is free: its readers finished before they signalled h_full of the previous block,
                // and this thread waited for that before phase 2 of the previous block)
                for (int kb = 0; kb < p.nk1; ++kb) {
                    if (!ptx::mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
                    ptx::tc_fence_after();
                    const uint64_t da = ptx::make_kmajor_sw128_desc(ptx::smem_u32(smem_a + stage * A_BYTES));
                    const uint64_t db = ptx::make_kmajor_sw128_desc(ptx::smem_u32(smem_b + stage * B_BYTES));
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)  // +32 bytes per 16-element K step, in the descriptor's 16-byte units
                        ptx::mma_f16_ss(tmem_base, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc1, (kb | k) != 0 ? 1u : 0u);
                    ptx::tc_commit(&empty_bar[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                ptx::tc_commit(acc1_full);
                // phase 2: the hidden block must be in shared memory, and acc2 drained by the previous block's epilogue
                if (!ptx::mbar_wait_bounded(h_full, blk & 1u, abort_flag)) { ok = false; break; }
                if (!ptx::mbar_wait_bounded(acc2_empty, (blk & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                ptx::tc_fence_after();
                for (int kb = 0; kb < p.nk2; ++kb) {
                    if (!ptx::mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
                    ptx::tc_fence_after();
                    const uint64_t da = ptx::make_kmajor_sw128_desc(h_addr + (uint32_t)(kb * A_BYTES));
                    const uint64_t db = ptx::make_kmajor_sw128_desc(ptx::smem_u32(smem_b + stage * B_BYTES));
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        ptx::mma_f16_ss(tmem_base + MAX_N, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc2, (kb | k) != 0 ? 1u : 0u);
                    ptx::tc_commit(&empty_bar[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                ptx::tc_commit(acc2_full);
            }
            if (!ok) {
                atomicOr(&g_mlp_status[0], 2u);
                // Let the MMAs already issued finish before TMEM is released.
                ptx::tc_commit(drain_bar);
                const uint64_t t0 = ptx::globaltimer_ns();
                while (!ptx::mbar_try_wait(drain_bar, 0)) {
                    if (ptx::globaltimer_ns() - t0 > ptx::kWaitLimitNs) break;
                }
            }
        }
    } else {
        // ------------------------------ epilogue warps ----------------------------
        const int quad = warp & 3;         // TMEM lanes [32*quad, 32*quad + 32) belong to this warp
        const int part = (warp - 2) >> 2;  // which of the quadrant's EPI_WARPS / 4 warps: they share the columns
        constexpr int PARTS = EPI_WARPS / 4;
        const int r = quad * 32 + lane;
        const uint32_t lane_field = (uint32_t)(quad * 32) << 16;
        const uint32_t h_row = ptx::smem_u32(smem_h) + (uint32_t)(r * 128);
        T* out = reinterpret_cast<T*>(p.out);
        const T* b1 = reinterpret_cast<const T*>(p.b1);
        const T* b2 = reinterpret_cast<const T*>(p.b2);
        uint32_t blk = 0;
        bool ok = true;
        for (int mb = blockIdx.x; mb < p.num_m_blocks && ok; mb += gridDim.x, ++blk) {
            // ---- hidden block: acc1 -> + b1, act1 -> 16-bit -> shared memory (K-major, 128-byte swizzle) ----
            // warp-uniform wait result: the TMEM loads below are warp-collective
            if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(acc1_full, blk & 1u, abort_flag))) { ok = false; break; }
            ptx::tc_fence_after();
            for (int q = part; q < 2 * p.nk2; q += PARTS) {  // 32-column chunks of every 64-column slab phase 2 will read
                const int col0 = q * 32;
                float v[32];
                if (col0 < p.n1p) {
                    uint32_t raw[32];
                    ptx::tmem_ld_32x32(tmem_base + lane_field + (uint32_t)col0, raw);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]);
                    finish_chunk<T>(v, b1, p.b1_vec_ok != 0, col0, p.N1, p.act1);
                    if (col0 + 32 > p.N1) {  // columns beyond the layer's width: zeros, whatever act1(0) is
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (col0 + i >= p.N1) v[i] = 0.f;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0.f;
                }
                const uint32_t slab = h_row + (uint32_t)((q >> 1) * A_BYTES);
#pragma unroll
                for (int t4 = 0; t4 < 4; ++t4) {
                    uint32_t w[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) w[i] = ptx::pack2<T>(v[t4 * 8 + 2 * i], v[t4 * 8 + 2 * i + 1]);
                    const int piece = (q & 1) * 4 + t4;  // 16-byte piece of this row's 128-byte segment
                    ptx::st_shared_v4(slab + (uint32_t)((piece ^ (r & 7)) << 4), make_uint4(w[0], w[1], w[2], w[3]));
                }
            }
            // the writes above must be visible to the tensor core's (async proxy) reads of shared memory
            ptx::fence_proxy_async();
            ptx::tc_fence_before();
            ptx::mbar_arrive(h_full);
            // ---- output block: acc2 -> + b2, act2 -> out ----
            if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(acc2_full, blk & 1u, abort_flag))) { ok = false; break; }
            ptx::tc_fence_after();
            const int64_t row = (int64_t)mb * BM + r;
            const bool row_ok = row < p.M;
            for (int col0 = part * 32; col0 < p.N2; col0 += PARTS * 32) {
                uint32_t raw[32];
                ptx::tmem_ld_32x32(tmem_base + lane_field + (uint32_t)(MAX_N + col0), raw);
                ptx::tmem_ld_wait();
                float v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]);
                finish_chunk<T>(v, b2, p.b2_vec_ok != 0, col0, p.N2, p.act2);
                if (!row_ok) continue;
                T* orow = out + row * p.ldc + col0;
                if (col0 + 32 <= p.N2 && p.out_vec_ok) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        Vec16<T> ov;
#pragma unroll
                        for (int j = 0; j < 8; ++j) ov.v[j] = Cvt<T>::from_f(v[i + j]);
                        st16(orow + i, ov);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (col0 + i < p.N2) orow[i] = Cvt<T>::from_f(v[i]);
                }
            }
            // all of this warp's reads of acc2 are complete (wait::ld above): the next block may overwrite it
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(acc2_empty);
        }
        if (!ok && lane == 0) atomicOr(&g_mlp_status[0], 4u);
    }

    // ------------------------------ teardown --------------------------------------
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <typename T>
int launch_mlp2(const void* x, const void* w1, const void* b1, const void* w2, const void* b2, void* out, int64_t M,
                int64_t K1, int64_t N1, int64_t N2, int64_t lda, int64_t ldw1, int64_t ldw2, int64_t ldc, int act1,
                int act2, cudaStream_t st) {
    constexpr bool is_bf16 = std::is_same<T, __nv_bfloat16>::value;
    MlpParams p;
    p.out = out;
    p.b1 = b1;
    p.b2 = b2;
    p.M = M;
    p.ldc = ldc;
    p.N1 = (int)N1;
    p.N2 = (int)N2;
    p.n1p = (int)((N1 + 15) / 16 * 16);
    p.n2p = (int)((N2 + 15) / 16 * 16);
    p.nk1 = (int)((K1 + BK - 1) / BK);
    p.nk2 = (int)((N1 + BK - 1) / BK);
    p.num_m_blocks = (int)((M + BM - 1) / BM);
    p.act1 = act1;
    p.act2 = act2;
    p.out_vec_ok = (aligned16(out) && ldc % 8 == 0) ? 1 : 0;
    p.b1_vec_ok = (b1 != nullptr && aligned16(b1)) ? 1 : 0;
    p.b2_vec_ok = (b2 != nullptr && aligned16(b2)) ? 1 : 0;
    CUtensorMap tx, tw1, tw2;
    if (!make_tmap_2d_16bit(&tx, x, (uint64_t)M, (uint64_t)K1, (uint64_t)lda, BM, BK, is_bf16) ||
        !make_tmap_2d_16bit(&tw1, w1, (uint64_t)N1, (uint64_t)K1, (uint64_t)ldw1, (uint32_t)p.n1p, BK, is_bf16) ||
        !make_tmap_2d_16bit(&tw2, w2, (uint64_t)N2, (uint64_t)N1, (uint64_t)ldw2, (uint32_t)p.n2p, BK, is_bf16))
        return fail(XG_ERR_UNSUPPORTED, "xg_mlp2_bias_act: tensor-map encoding failed");
    auto kern = mlp2_kernel<T>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, MLP_SMEM_BYTES);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(XG_ERR_LAUNCH, "xg_mlp2_bias_act: cannot reserve shared memory: %s", cudaGetErrorString(e));
    }
    const int sms = num_sms();
    const unsigned grid = (unsigned)(p.num_m_blocks < sms ? p.num_m_blocks : sms);
    kern<<<grid, MLP_THREADS, MLP_SMEM_BYTES, st>>>(tx, tw1, tw2, p);
    return check_launch("xg_mlp2_bias_act");
}

}  // namespace

int read_mlp_status(unsigned int* host_out, int reset) {
    unsigned int v[4] = {0, 0, 0, 0};
    if (cudaMemcpyFromSymbol(v, g_mlp_status, sizeof(v)) != cudaSuccess) {
        cudaGetLastError();
        return fail(XG_ERR_DEVICE, "xg_tc_status: cannot read device status");
    }
    *host_out = v[0];
    if (reset && v[0] != 0) {
        unsigned int z[4] = {0, 0, 0, 0};
        cudaMemcpyToSymbol(g_mlp_status, z, sizeof(z));
    }
    return XG_OK;
}

}  // namespace xg

extern "C" int xg_mlp2_supported(int64_t M, int64_t K1, int64_t N1, int64_t N2, int dtype) {
    return (dtype == XG_BF16 || dtype == XG_F16) && M > 0 && K1 >= 8 && K1 % 8 == 0 && N1 >= 16 && N1 <= xg::MAX_N &&
                   N1 % 8 == 0 && N2 >= 1 && N2 <= xg::MAX_N && M < (int64_t)xg::BM * 0x7fffff
               ? 1
               : 0;
}

extern "C" int xg_mlp2_bias_act(const void* x, const void* w1, const void* b1, const void* w2, const void* b2, void* out,
                                int64_t M, int64_t K1, int64_t N1, int64_t N2, int64_t lda, int64_t ldw1, int64_t ldw2,
                                int64_t ldc, int act1, int act2, int dtype, void* stream) {
    using namespace xg;
    if (!x || !w1 || !w2 || !out) return fail(XG_ERR_INVALID_ARG, "xg_mlp2_bias_act: null pointer");
    if (M < 0 || K1 <= 0 || N1 <= 0 || N2 <= 0) return fail(XG_ERR_INVALID_ARG, "xg_mlp2_bias_act: bad extents");
    if (act1 < XG_ACT_NONE || act1 > XG_ACT_SIGMOID || act2 < XG_ACT_NONE || act2 > XG_ACT_SIGMOID)
        return fail(XG_ERR_INVALID_ARG, "xg_mlp2_bias_act: bad activation code");
    if (M == 0) return XG_OK;
    if (!xg_mlp2_supported(M, K1, N1, N2, dtype))
        return fail(XG_ERR_UNSUPPORTED,
                    "xg_mlp2_bias_act: needs a 16-bit dtype, K1 %% 8 == 0, 16 <= N1 <= 256 with N1 %% 8 == 0 and N2 <= 256 "
                    "(got K1 %lld, N1 %lld, N2 %lld, dtype %d)", (long long)K1, (long long)N1, (long long)N2, dtype);
    if (lda < K1 || ldw1 < K1 || ldw2 < N1 || ldc < N2) return fail(XG_ERR_INVALID_ARG, "xg_mlp2_bias_act: a row stride is shorter than its row");
    if (!aligned16(x) || !aligned16(w1) || !aligned16(w2) || lda % 8 != 0 || ldw1 % 8 != 0 || ldw2 % 8 != 0)
        return fail(XG_ERR_UNSUPPORTED, "xg_mlp2_bias_act: x, W1 and W2 must be 16-byte aligned with row strides that are multiples of 8 elements");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (dtype == XG_BF16)
        return launch_mlp2<__nv_bfloat16>(x, w1, b1, w2, b2, out, M, K1, N1, N2, lda, ldw1, ldw2, ldc, act1, act2, st);
    return launch_mlp2<__half>(x, w1, b1, w2, b2, out, M, K1, N1, N2, lda, ldw1, ldw2, ldc, act1, act2, st);
}
