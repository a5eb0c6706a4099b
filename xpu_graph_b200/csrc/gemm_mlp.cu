// Two or three chained dense layers in one kernel: out = act_L(... act1(x W1^T + b1) ... W_L^T + b_L) for narrow 16-bit
// layers (every width <= 256), the place of the reference's serial-matmul kernels (targets/mlu/fuse_densetower.py:272-316,
// triton_kernel/fused_serial_mm_2dot.py:142, fused_serial_mm_3dot.py:271): the hidden activations never leave the SM.
//
// One persistent CTA per SM walks 128-row blocks of x. Per block and layer l:
//   product   acc[128 x N_l] = a W_l^T  (tcgen05.mma). Layer 1 streams x and W1 by TMA through a 3-stage ring; later
//             layers read a = the previous hidden block from shared memory and stream only W_l through the same ring.
//   hand-over (hidden layers) the eight epilogue warps read acc from TMEM, add b_l, apply act_l, round to the 16-bit type
//             (the rounding the unfused graph does when it stores the hidden tensor) and write the result into shared
//             memory in the K-major 128-byte-swizzled layout an MMA A operand wants (the layout TMA would have produced)
//   epilogue  (last layer) acc + b_L, act_L -> out
// The accumulators alternate between two TMEM regions, so with two layers the first product of the next block runs
// while the epilogue of the current one drains. One hidden buffer is enough for any depth: a layer's product has
// completed (and with it every read of the buffer) before that layer's own hand-over writes it. Ragged extents need no
// special code: TMA zero-fills outside the tensors, hidden columns beyond a layer's width are written as zeros, rows
// beyond M are not stored.
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
constexpr int EPI_WARPS = 8;                // two per TMEM lane quadrant (a single warp per scheduler is latency-bound):
                                            // warp part p of a quadrant takes the 32-column chunks q = p, p + 2, ...
constexpr int MLP_THREADS = 64 + EPI_WARPS * 32;  // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue
constexpr int TMEM_COLS = 512;              // acc1 [0, 256), acc2 [256, 512)

constexpr int MAX_LAYERS = 3;

struct MlpParams {
    void* out;
    const void* bias[MAX_LAYERS];
    int64_t M, ldc;
    int layers;                  // 2 or 3
    int num_m_blocks;
    int N[MAX_LAYERS];           // layer widths
    int np[MAX_LAYERS];          // MMA N of each product: the width rounded up to 16
    int nk[MAX_LAYERS];          // 64-column k-blocks of each product (over K1 for layer 1, over N_{l-1} after)
    int act[MAX_LAYERS];
    int bias_vec_ok;             // bit l: bias l allows 16-byte loads
    int w_kn;                    // bit l: weight l is stored [K, N] (consumed MN-major) instead of [N, K]
    int out_vec_ok;              // out and ldc allow 16-byte stores
};
static_assert(sizeof(MlpParams) <= 128, "the scalar parameters stay within 128 bytes beside the tensor maps");

__device__ __forceinline__ float apply_act(float v, int act) {
    switch (act) {
        case XG_ACT_GELU: return gelu_erf_16bit(v);  // results of this file are always rounded to a 16-bit type
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
mlp_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w1,
           const __grid_constant__ CUtensorMap tmap_w2, const __grid_constant__ CUtensorMap tmap_w3, const __grid_constant__ MlpParams p) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: required by the 128-byte swizzle pattern shared by TMA and the MMA descriptors.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;                           // [STAGES][A_BYTES]
    uint8_t* smem_b = smem + STAGES * A_BYTES;        // [STAGES][B_BYTES]
    uint8_t* smem_h = smem + STAGES * STAGE_BYTES;    // [H_SLABS][A_BYTES]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_h + H_BYTES);
    uint64_t* full_bar = bars;                // [STAGES]
    uint64_t* empty_bar = bars + STAGES;      // [STAGES]
    uint64_t* acc_full = bars + 2 * STAGES;   // [2] a product into this accumulator region has completed
    uint64_t* acc_empty = acc_full + 2;       // [2] the epilogue warps have read the region (one arrival per warp)
    uint64_t* h_full = acc_full + 4;          // [H_SLABS] a 64-column slab of a hidden block is in shared memory (every
                                              // epilogue thread writes 32 columns of each slab and arrives once per slab)
    uint64_t* drain_bar = h_full + H_SLABS;
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        for (int r = 0; r < 2; ++r) {
            ptx::mbar_init(&acc_full[r], 1);
            ptx::mbar_init(&acc_empty[r], EPI_WARPS);
        }
        for (int c = 0; c < H_SLABS; ++c) ptx::mbar_init(&h_full[c], EPI_WARPS * 32);
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

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (ptx::elect_one()) {
            ptx::prefetch_tensormap(&tmap_x);
            ptx::prefetch_tensormap(&tmap_w1);
            ptx::prefetch_tensormap(&tmap_w2);
            if (p.layers > 2) ptx::prefetch_tensormap(&tmap_w3);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t armed = 0, armed_phase = 0;  // stages with a load of this thread in flight, and the parity of each
            bool ok = true;
            for (int mb = blockIdx.x; mb < p.num_m_blocks && ok; mb += gridDim.x) {
                for (int l = 0; l < p.layers && ok; ++l) {
                    const CUtensorMap* tw = l == 0 ? &tmap_w1 : (l == 1 ? &tmap_w2 : &tmap_w3);
                    // [N, K] weights: one box of np rows x 64 k-columns. [K, N] weights: boxes of 64 k-rows x 64 n-columns,
                    // one per 64 output columns, which the MMA consumes MN-major exactly as TMA leaves them.
                    const bool kn = (p.w_kn >> l) & 1;
                    const int n_boxes = (p.np[l] + 63) / 64;
                    const uint32_t w_bytes = kn ? (uint32_t)n_boxes * (BK * 128) : (uint32_t)p.np[l] * BK * 2;
                    for (int kb = 0; kb < p.nk[l]; ++kb) {
                        if (!ptx::mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
                        if (l == 0) {
                            ptx::mbar_arrive_expect_tx(&full_bar[stage], A_BYTES + w_bytes);
                            ptx::tma_load_2d(smem_a + stage * A_BYTES, &tmap_x, &full_bar[stage], kb * BK, mb * BM);
                        } else {
                            ptx::mbar_arrive_expect_tx(&full_bar[stage], w_bytes);
                        }
                        if (kn) {
                            for (int jn = 0; jn < n_boxes; ++jn)
                                ptx::tma_load_2d(smem_b + stage * B_BYTES + jn * (BK * 128), tw, &full_bar[stage], jn * 64, kb * BK);
                        } else {
                            ptx::tma_load_2d(smem_b + stage * B_BYTES, tw, &full_bar[stage], kb * BK, 0);
                        }
                        armed |= 1u << stage;
                        armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
                        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                    }
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
            const uint32_t h_addr = ptx::smem_u32(smem_h);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t uses0 = 0, uses1 = 0;  // products issued into each accumulator region so far
            uint32_t hand_par = 0;      // bit c: parity of slab barrier c's next phase (hand-overs differ in their slab counts)
            bool ok = true;
            for (int mb = blockIdx.x; mb < p.num_m_blocks && ok; mb += gridDim.x) {
                for (int l = 0; l < p.layers && ok; ++l) {
                    const int r = l & 1;
                    const bool kn = (p.w_kn >> l) & 1;
                    const uint32_t idesc = ptx::make_idesc_f16(fmt, BM, p.np[l], kn ? 1 : 0);
                    // the region's previous product has been read by the epilogue warps
                    if (!ptx::mbar_wait_bounded(&acc_empty[r], ((r ? uses1 : uses0) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                    ptx::tc_fence_after();
                    for (int kb = 0; kb < p.nk[l]; ++kb) {
                        // slab kb of the previous layer's result is in shared memory (the slabs arrive in order, so the
                        // product starts while the later ones are still being written)
                        if (l > 0) {
                            if (!ptx::mbar_wait_bounded(&h_full[kb], (hand_par >> kb) & 1u, abort_flag)) { ok = false; break; }
                            hand_par ^= 1u << kb;
                        }
                        if (!ptx::mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
                        ptx::tc_fence_after();
                        const uint64_t da = ptx::make_kmajor_sw128_desc(l == 0 ? ptx::smem_u32(smem_a + stage * A_BYTES)
                                                                                : h_addr + (uint32_t)(kb * A_BYTES));
                        const uint32_t b_addr = ptx::smem_u32(smem_b + stage * B_BYTES);
                        const uint64_t db = kn ? ptx::make_mnmajor_sw128_desc(b_addr, BK * 128) : ptx::make_kmajor_sw128_desc(b_addr);
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)  // per 16-element K step: K-major +32 bytes, MN-major +16 rows of 128
                                                           // bytes (both in the descriptor's 16-byte units)
                            ptx::mma_f16_ss(tmem_base + (uint32_t)(r * MAX_N), da + (uint64_t)(k * 2), db + (uint64_t)(kn ? k * 128 : k * 2),
                                            idesc, (kb | k) != 0 ? 1u : 0u);
                        ptx::tc_commit(&empty_bar[stage]);
                        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                    }
                    if (!ok) break;
                    ptx::tc_commit(&acc_full[r]);
                    if (r) ++uses1; else ++uses0;
                }
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
        const int r_in_blk = quad * 32 + lane;
        const uint32_t lane_field = (uint32_t)(quad * 32) << 16;
        const uint32_t h_row = ptx::smem_u32(smem_h) + (uint32_t)(r_in_blk * 128);
        T* out = reinterpret_cast<T*>(p.out);
        uint32_t uses0 = 0, uses1 = 0;  // products consumed from each accumulator region so far
        bool ok = true;
        for (int mb = blockIdx.x; mb < p.num_m_blocks && ok; mb += gridDim.x) {
            for (int l = 0; l < p.layers && ok; ++l) {
                const int r = l & 1;
                const T* bias = reinterpret_cast<const T*>(p.bias[l]);
                const uint32_t acc = tmem_base + lane_field + (uint32_t)(r * MAX_N);
                // warp-uniform wait result: the TMEM loads below are warp-collective
                if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(&acc_full[r], (r ? uses1 : uses0) & 1u, abort_flag))) { ok = false; break; }
                if (r) ++uses1; else ++uses0;
                ptx::tc_fence_after();
                if (l + 1 < p.layers) {
                    // ---- hidden block: acc -> + bias, act -> 16-bit -> shared memory (K-major, 128-byte swizzle) ----
                    for (int q = part; q < 2 * p.nk[l + 1]; q += PARTS) {  // 32-column chunks of every slab the next product reads
                        const int col0 = q * 32;
                        float v[32];
                        if (col0 < p.np[l]) {
                            uint32_t raw[32];
                            ptx::tmem_ld_32x32(acc + (uint32_t)col0, raw);
                            ptx::tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]);
                            finish_chunk<T>(v, bias, ((p.bias_vec_ok >> l) & 1) != 0, col0, p.N[l], p.act[l]);
                            if (col0 + 32 > p.N[l]) {  // columns beyond the layer's width: zeros, whatever act(0) is
#pragma unroll
                                for (int i = 0; i < 32; ++i)
                                    if (col0 + i >= p.N[l]) v[i] = 0.f;
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
                            ptx::st_shared_v4(slab + (uint32_t)((piece ^ (r_in_blk & 7)) << 4), make_uint4(w[0], w[1], w[2], w[3]));
                        }
                        // this thread's part of slab q / 2 must be visible to the tensor core's (async proxy) reads
                        ptx::fence_proxy_async();
                        ptx::mbar_arrive(&h_full[q >> 1]);
                    }
                    ptx::tc_fence_before();
                } else {
                    // ---- output block: acc -> + bias, act -> out ----
                    const int64_t row = (int64_t)mb * BM + r_in_blk;
                    const bool row_ok = row < p.M;
                    for (int col0 = part * 32; col0 < p.N[l]; col0 += PARTS * 32) {
                        uint32_t raw[32];
                        ptx::tmem_ld_32x32(acc + (uint32_t)col0, raw);
                        ptx::tmem_ld_wait();
                        float v[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]);
                        finish_chunk<T>(v, bias, ((p.bias_vec_ok >> l) & 1) != 0, col0, p.N[l], p.act[l]);
                        if (!row_ok) continue;
                        T* orow = out + row * p.ldc + col0;
                        if (col0 + 32 <= p.N[l] && p.out_vec_ok) {
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
                                if (col0 + i < p.N[l]) orow[i] = Cvt<T>::from_f(v[i]);
                        }
                    }
                    ptx::tc_fence_before();
                }
                // all of this warp's reads of the region are complete (wait::ld above): a later product may overwrite it
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&acc_empty[r]);
            }
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
int launch_mlp(const char* who, const void* x, int layers, const void* const* w, const void* const* b, void* out, int64_t M,
               int64_t K1, const int64_t* N, int64_t lda, const int64_t* ldw, int64_t ldc, const int* act, int weights_kn,
               cudaStream_t st) {
    constexpr bool is_bf16 = std::is_same<T, __nv_bfloat16>::value;
    MlpParams p;
    p.out = out;
    p.M = M;
    p.ldc = ldc;
    p.layers = layers;
    p.num_m_blocks = (int)((M + BM - 1) / BM);
    p.out_vec_ok = (aligned16(out) && ldc % 8 == 0) ? 1 : 0;
    p.bias_vec_ok = 0;
    p.w_kn = 0;
    CUtensorMap tx, tw[MAX_LAYERS];
    bool maps_ok = make_tmap_2d_16bit(&tx, x, (uint64_t)M, (uint64_t)K1, (uint64_t)lda, BM, BK, is_bf16);
    for (int l = 0; l < MAX_LAYERS; ++l) {
        const int s = l < layers ? l : layers - 1;  // an unused slot repeats the last layer: the kernel never reads it
        const int64_t k = s == 0 ? K1 : N[s - 1];
        p.bias[l] = b[s];
        p.N[l] = (int)N[s];
        p.np[l] = (int)((N[s] + 15) / 16 * 16);
        p.nk[l] = (int)((k + BK - 1) / BK);
        p.act[l] = act[s];
        if (b[s] != nullptr && aligned16(b[s])) p.bias_vec_ok |= 1 << l;
        if ((weights_kn >> s) & 1) {
            p.w_kn |= 1 << l;
            maps_ok = maps_ok && make_tmap_2d_16bit(&tw[l], w[s], (uint64_t)k, (uint64_t)N[s], (uint64_t)ldw[s], BK, 64, is_bf16);
        } else {
            maps_ok = maps_ok && make_tmap_2d_16bit(&tw[l], w[s], (uint64_t)N[s], (uint64_t)k, (uint64_t)ldw[s], (uint32_t)p.np[l], BK, is_bf16);
        }
    }
    if (!maps_ok) return fail(XG_ERR_UNSUPPORTED, "%s: tensor-map encoding failed", who);
    auto kern = mlp_kernel<T>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, MLP_SMEM_BYTES);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(XG_ERR_LAUNCH, "%s: cannot reserve shared memory: %s", who, cudaGetErrorString(e));
    }
    const int sms = num_sms();
    const unsigned grid = (unsigned)(p.num_m_blocks < sms ? p.num_m_blocks : sms);
    kern<<<grid, MLP_THREADS, MLP_SMEM_BYTES, st>>>(tx, tw[0], tw[1], tw[2], p);
    return check_launch(who);
}

bool mlp_supported(int64_t M, int64_t K1, int layers, const int64_t* N, int dtype) {
    if (!(dtype == XG_BF16 || dtype == XG_F16) || M <= 0 || M >= (int64_t)BM * 0x7fffff || K1 < 8 || K1 % 8 != 0) return false;
    for (int l = 0; l < layers; ++l) {
        if (N[l] < 1 || N[l] > MAX_N) return false;
        if (l + 1 < layers && (N[l] < 16 || N[l] % 8 != 0)) return false;  // a hidden width is the next product's K
    }
    return true;
}

int mlp_entry(const char* who, const void* x, int layers, const void* const* w, const void* const* b, void* out, int64_t M,
              int64_t K1, const int64_t* N, int64_t lda, const int64_t* ldw, int64_t ldc, const int* act, int weights_kn,
              int dtype, void* stream) {
    if (!x || !out) return fail(XG_ERR_INVALID_ARG, "%s: null pointer", who);
    if (M < 0 || K1 <= 0) return fail(XG_ERR_INVALID_ARG, "%s: bad extents", who);
    for (int l = 0; l < layers; ++l) {
        if (!w[l]) return fail(XG_ERR_INVALID_ARG, "%s: null weight pointer", who);
        if (N[l] <= 0) return fail(XG_ERR_INVALID_ARG, "%s: bad extents", who);
        if (act[l] < XG_ACT_NONE || act[l] > XG_ACT_SIGMOID) return fail(XG_ERR_INVALID_ARG, "%s: bad activation code", who);
    }
    if (M == 0) return XG_OK;
    if (!mlp_supported(M, K1, layers, N, dtype))
        return fail(XG_ERR_UNSUPPORTED,
                    "%s: needs a 16-bit dtype, K1 %% 8 == 0, every width <= 256 and hidden widths >= 16 that are multiples of 8 "
                    "(got K1 %lld, N1 %lld, N2 %lld, dtype %d)", who, (long long)K1, (long long)N[0], (long long)N[1], dtype);
    if (lda < K1 || ldc < N[layers - 1]) return fail(XG_ERR_INVALID_ARG, "%s: a row stride is shorter than its row", who);
    if (!aligned16(x) || lda % 8 != 0)
        return fail(XG_ERR_UNSUPPORTED, "%s: x must be 16-byte aligned with a row stride that is a multiple of 8 elements", who);
    if (weights_kn < 0 || weights_kn >= (1 << layers)) return fail(XG_ERR_INVALID_ARG, "%s: bad weight layout mask", who);
    for (int l = 0; l < layers; ++l) {
        const bool kn = (weights_kn >> l) & 1;  // rows of a [K, N] weight are N long
        if (ldw[l] < (kn ? N[l] : (l == 0 ? K1 : N[l - 1]))) return fail(XG_ERR_INVALID_ARG, "%s: a row stride is shorter than its row", who);
        if (!aligned16(w[l]) || ldw[l] % 8 != 0)
            return fail(XG_ERR_UNSUPPORTED, "%s: weights must be 16-byte aligned with row strides that are multiples of 8 elements", who);
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (dtype == XG_BF16) return launch_mlp<__nv_bfloat16>(who, x, layers, w, b, out, M, K1, N, lda, ldw, ldc, act, weights_kn, st);
    return launch_mlp<__half>(who, x, layers, w, b, out, M, K1, N, lda, ldw, ldc, act, weights_kn, st);
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
    const int64_t N[2] = {N1, N2};
    return xg::mlp_supported(M, K1, 2, N, dtype) ? 1 : 0;
}

extern "C" int xg_mlp3_supported(int64_t M, int64_t K1, int64_t N1, int64_t N2, int64_t N3, int dtype) {
    const int64_t N[3] = {N1, N2, N3};
    return xg::mlp_supported(M, K1, 3, N, dtype) ? 1 : 0;
}

extern "C" int xg_mlp2_bias_act(const void* x, const void* w1, const void* b1, const void* w2, const void* b2, void* out,
                                int64_t M, int64_t K1, int64_t N1, int64_t N2, int64_t lda, int64_t ldw1, int64_t ldw2,
                                int64_t ldc, int act1, int act2, int weights_kn, int dtype, void* stream) {
    const void* w[2] = {w1, w2};
    const void* b[2] = {b1, b2};
    const int64_t N[2] = {N1, N2}, ldw[2] = {ldw1, ldw2};
    const int act[2] = {act1, act2};
    return xg::mlp_entry("xg_mlp2_bias_act", x, 2, w, b, out, M, K1, N, lda, ldw, ldc, act, weights_kn, dtype, stream);
}

extern "C" int xg_mlp3_bias_act(const void* x, const void* w1, const void* b1, const void* w2, const void* b2, const void* w3,
                                const void* b3, void* out, int64_t M, int64_t K1, int64_t N1, int64_t N2, int64_t N3,
                                int64_t lda, int64_t ldw1, int64_t ldw2, int64_t ldw3, int64_t ldc, int act1, int act2,
                                int act3, int weights_kn, int dtype, void* stream) {
    const void* w[3] = {w1, w2, w3};
    const void* b[3] = {b1, b2, b3};
    const int64_t N[3] = {N1, N2, N3}, ldw[3] = {ldw1, ldw2, ldw3};
    const int act[3] = {act1, act2, act3};
    return xg::mlp_entry("xg_mlp3_bias_act", x, 3, w, b, out, M, K1, N, lda, ldw, ldc, act, weights_kn, dtype, stream);
}
