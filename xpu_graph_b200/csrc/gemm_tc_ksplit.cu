// Dense layer for problems with few output tiles (small M: the weight-streaming regime), 16-bit inputs.
//
// A 256 x 256 output tile belongs to a thread-block cluster of 2*S CTAs = S CTA pairs. Pair s computes the tile over
// its share of the k-blocks with tcgen05.mma.cta_group::2 (each CTA loads 128 activation rows and 128 weight rows per
// k-block, fp32 accumulators in TMEM), so every weight element enters exactly one SM once and the activations enter
// S times fewer SMs than with independent 128-row CTAs. The S partial tiles are then added through distributed shared
// memory: the tile's columns are dealt out to the pairs; each CTA sends the columns it does not own from TMEM through
// registers straight into their owner's receive area (st.async to shared::cluster, 16 bytes per message, completion
// counted in bytes on the owner's mbarrier), and the owner adds the partials in split order (deterministic), applies
// bias / residual / activation and stores. No global scratch memory, no second launch, no atomics.
//
// Warp roles per CTA: warp 0 = TMA producer, warp 1 = MMA issuer (leader CTA of the pair only), warps 2..17 = epilogue
// (a warp reads the 32 accumulator rows of its TMEM lane quadrant, 16 columns at a time; the four warps of a quadrant
// share out the columns). Every TMA load is issued by the CTA that consumes it (no cluster multicast).
#include "common.cuh"
#include "sm100_ptx.cuh"

#include <cstdlib>
#include <cstring>
#include <type_traits>

namespace xg {

__device__ unsigned int g_ksplit_status[4];

namespace {

constexpr int BM = 128;        // rows per CTA (a pair covers 256)
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int TILE = 256;      // activation rows of a tile, and the widest tile (weight rows)
constexpr int KS_EPI_WARPS = 16;  // four per TMEM lane quadrant: a lone warp per scheduler would run at instruction latency
constexpr int KS_THREADS = 64 + KS_EPI_WARPS * 32;
constexpr int KS_STAGES_SPLIT = 4;  // pipeline depth when the receive area is needed (S > 1)
constexpr int KS_STAGES_WHOLE = 7;  // ... and when the whole of shared memory is the pipeline (S = 1)
constexpr int KS_STAGE_BYTES = 2 * BM * BK * 2;   // per CTA: 128 activation rows + up to 128 weight rows = 32 KiB
constexpr int KS_CHUNK_BYTES = BM * 32 * 4;       // one 32-column chunk of a CTA's 128 rows in fp32 = 16 KiB
constexpr int KS_RECV_CHUNKS = 6;                 // (S - 1) senders x owned chunks: 3 x 2 (S = 4), 2 x 3 (S = 3), 1 x 4 (S = 2)
constexpr int KS_SMEM_BYTES = KS_STAGES_SPLIT * KS_STAGE_BYTES + KS_RECV_CHUNKS * KS_CHUNK_BYTES + 1024 /*alignment slack*/ +
                              256 /*barriers*/ + TILE * 4 /*the tile's bias row in fp32*/;
constexpr int KS_MAX_SPLIT = 4;

struct KsplitParams {
    void* out;
    const void* bias;
    const void* residual;
    int64_t M, N, ldc, ldr;
    int act;
    int vec_ok;       // out (and residual) rows are 16-byte addressable
    int bias_vec_ok;  // bias pointer 16-byte aligned
    int num_m_blocks, num_n_blocks, num_k_blocks;
    int S;            // pairs per cluster = k-splits
    int tn;           // tile width (weight rows per tile): a multiple of 32 in [64, 256], at least 32 * S
    int stages;       // pipeline depth
};
static_assert(KS_SMEM_BYTES <= 232448, "shared memory of one CTA");
static_assert(KS_STAGES_WHOLE * KS_STAGE_BYTES <= KS_STAGES_SPLIT * KS_STAGE_BYTES + KS_RECV_CHUNKS * KS_CHUNK_BYTES, "S = 1 layout");
static_assert(sizeof(KsplitParams) <= 128, "keep the kernel parameter block within 512 bytes");

__device__ __forceinline__ float act_of(float v, int act) {
    switch (act) {
        case XG_ACT_GELU: return gelu_erf_16bit(v);  // results of this file are always rounded to a 16-bit type
        case XG_ACT_RELU: return v > 0.f ? v : 0.f;
        case XG_ACT_SILU: return __fdividef(v, 1.0f + __expf(-v));
        case XG_ACT_SIGMOID: return __fdividef(1.0f, 1.0f + __expf(-v));
        default: return v;
    }
}

// chunks [lo, hi) of the tile's nch 32-column chunks are finished by pair s
__device__ __forceinline__ int chunk_lo(int s, int S, int nch) { return (s * nch) / S; }

// 16 bytes from registers into a peer CTA's shared memory; the bytes are counted on the peer's mbarrier as they land.
__device__ __forceinline__ void st_async_v4(uint32_t peer_dst, uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t peer_bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
                 ::"r"(peer_dst), "r"(a), "r"(b), "r"(c), "r"(d), "r"(peer_bar)
                 : "memory");
}
__device__ __forceinline__ void epilogue_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(KS_EPI_WARPS * 32) : "memory"); }

// bias, residual, activation and store of 16 finished columns of one row
template <typename T>
__device__ __forceinline__ void store_cols16(const KsplitParams& p, float (&v)[16], const float* bias_s, int64_t row, bool row_ok,
                                             int64_t col0) {
    const T* resid = reinterpret_cast<const T*>(p.residual);
    T* out = reinterpret_cast<T*>(p.out);
    const bool full = (col0 + 16 <= p.N);
#pragma unroll
    for (int i = 0; i < 16; i += 4) {  // zero where there is no bias; the same address in all lanes
        const float4 b4 = *reinterpret_cast<const float4*>(bias_s + i);
        v[i] += b4.x; v[i + 1] += b4.y; v[i + 2] += b4.z; v[i + 3] += b4.w;
    }
    if (!row_ok) return;
    if (full && p.vec_ok) {
        if (resid != nullptr) {
            const T* rr = resid + row * p.ldr + col0;
#pragma unroll
            for (int i = 0; i < 16; i += 8) {
                const Vec16<T> rv = ld16_stream(rr + i);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[i + j] += Cvt<T>::to_f(rv.v[j]);
            }
        }
        T* orow = out + row * p.ldc + col0;
#pragma unroll
        for (int i = 0; i < 16; i += 8) {
            Vec16<T> ov;
#pragma unroll
            for (int j = 0; j < 8; ++j) ov.v[j] = Cvt<T>::from_f(act_of(v[i + j], p.act));
            st16(orow + i, ov);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (col0 + i < p.N) {
                float a = v[i];
                if (resid != nullptr) a += Cvt<T>::to_f(resid[row * p.ldr + col0 + i]);
                out[row * p.ldc + col0 + i] = Cvt<T>::from_f(act_of(a, p.act));
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(KS_THREADS, 1)
gemm_tc_ksplit_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                      const KsplitParams p) {
    constexpr int A_BYTES = BM * BK * 2;
    const int STAGES = p.stages;
    const int S = p.S;
    const int TN = p.tn, nch = TN / 32;
    const uint32_t w_bytes = (uint32_t)(TN / 2) * (BK * 2);  // this CTA's half of the W tile per k-block
    extern __shared__ uint8_t smem_raw[];
    // Every CTA of the cluster computes the same offset here (the dynamic window starts at the same shared-memory
    // address in all CTAs of a launch), so that addresses mapped into a peer CTA point at the same object there.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // stage i: [A tile 16 KiB][W half tile <= 16 KiB]; then (S > 1 only) the receive area; then the barriers
    uint8_t* recv = smem + KS_STAGES_SPLIT * KS_STAGE_BYTES;  // [KS_RECV_CHUNKS][8 float4 columns][128 rows][16 bytes]
    uint64_t* bars = reinterpret_cast<uint64_t*>(recv + KS_RECV_CHUNKS * KS_CHUNK_BYTES);
    uint64_t* full_bar = bars;        // [8]  (used in the pair's leader)
    uint64_t* empty_bar = bars + 8;   // [8]  (each CTA its own)
    uint64_t* tmem_full = bars + 16;  // [1]  (each CTA its own)
    uint64_t* recv_full = bars + 17;  // [1]  counts the bytes the other S - 1 pairs send
    uint64_t* drain_bar = bars + 18;  // [1]
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 19);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    float* bias_s = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);  // [TILE]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t crank = ptx::cluster_ctarank();  // 0 .. 2S-1
    const int s = (int)(crank >> 1);                // this pair's k-split
    const uint32_t r = crank & 1u;                  // 0 = leader of the pair
    const uint32_t leader = crank & ~1u;
    const int tile = (int)(blockIdx.x / (unsigned)(2 * S));
    const int mb = tile % p.num_m_blocks, nb = tile / p.num_m_blocks;
    int kb0, kb1;
    {
        const int nkb = p.num_k_blocks, base = nkb / S, rem = nkb % S;
        kb0 = s * base + (s < rem ? s : rem);
        kb1 = kb0 + base + (s < rem ? 1 : 0);
    }

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) {
            ptx::mbar_init(&full_bar[i], 1);
            ptx::mbar_init(&empty_bar[i], 1);
        }
        ptx::mbar_init(tmem_full, 1);
        ptx::mbar_init(recv_full, 1);
        // what the other pairs will send: (S - 1) senders x this pair's chunks, counted in bytes
        if (S > 1) ptx::mbar_arrive_expect_tx(recv_full, (uint32_t)((S - 1) * (chunk_lo(s + 1, S, nch) - chunk_lo(s, S, nch)) * KS_CHUNK_BYTES));
        ptx::mbar_init(drain_bar, 1);
        *abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::fence_proxy_async();
    }
    if (warp == 1) ptx::tmem_alloc_pair(tmem_base_slot, TILE);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();  // every CTA's barriers exist before anyone signals across the cluster
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == 0) {
        // ------------------------------ TMA producer (every CTA) ------------------------------
        if (ptx::elect_one()) {
            ptx::prefetch_tensormap(&tmap_a);
            ptx::prefetch_tensormap(&tmap_w);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!ptx::mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
                if (r == 0) ptx::mbar_arrive_expect_tx(&full_bar[stage], 2u * ((uint32_t)A_BYTES + w_bytes));
                const uint32_t full_leader = ptx::map_to_cta(ptx::smem_u32(&full_bar[stage]), leader);
                uint8_t* st = smem + stage * KS_STAGE_BYTES;
                ptx::tma_load_2d_pair(st, &tmap_a, full_leader, kb * BK, mb * TILE + (int)r * BM);
                ptx::tma_load_2d_pair(st + A_BYTES, &tmap_w, full_leader, kb * BK, nb * TN + (int)r * (TN / 2));
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (!ok) atomicOr(&g_ksplit_status[0], 1u);
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (leader CTA of each pair) ------------------
        if (r == 0 && ptx::elect_one()) {
            const uint32_t idesc = ptx::make_idesc_f16(std::is_same<T, __nv_bfloat16>::value ? 1 : 0, 256, TN, 0);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!ptx::mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
                ptx::tc_fence_after();
                const uint32_t st = ptx::smem_u32(smem + stage * KS_STAGE_BYTES);
                const uint64_t da = ptx::make_kmajor_sw128_desc(st);
                const uint64_t dw = ptx::make_kmajor_sw128_desc(st + A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    ptx::mma_f16_ss_pair(tmem_base, da + (uint64_t)(k * 2), dw + (uint64_t)(k * 2), idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
                const uint32_t e = ptx::smem_u32(&empty_bar[stage]);
                ptx::tc_commit_pair(ptx::map_to_cta(e, leader));
                ptx::tc_commit_pair(ptx::map_to_cta(e, leader + 1));
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (ok) {
                const uint32_t f = ptx::smem_u32(tmem_full);
                ptx::tc_commit_pair(ptx::map_to_cta(f, leader));
                ptx::tc_commit_pair(ptx::map_to_cta(f, leader + 1));
            } else {
                atomicOr(&g_ksplit_status[0], 2u);
                ptx::tc_commit_pair(ptx::map_to_cta(ptx::smem_u32(drain_bar), leader));
                const uint64_t t0 = ptx::globaltimer_ns();
                while (!ptx::mbar_try_wait(drain_bar, 0)) {
                    if (ptx::globaltimer_ns() - t0 > ptx::kWaitLimitNs) break;
                }
            }
        }
    } else {
        // ------------------------------ epilogue (every CTA) ----------------------------------
        const int quad = warp & 3;          // TMEM lanes [32 quad, 32 quad + 32) are the ones this warp may read
        const int grp = (warp - 2) >> 2;    // 0..3: which share of the columns this warp takes within its quadrant
        constexpr int GROUPS = KS_EPI_WARPS / 4;
        const int row_in_cta = quad * 32 + lane;
        const int64_t row = (int64_t)mb * TILE + (int64_t)r * BM + row_in_cta;
        const uint32_t lane_field = (uint32_t)(quad * 32) << 16;
        const uint32_t recv_row = ptx::smem_u32(recv) + (uint32_t)(row_in_cta * 16);
        const int my_lo = chunk_lo(s, S, nch), my_hi = chunk_lo(s + 1, S, nch), mine = my_hi - my_lo;
        // the tile's bias row, once, while the main loop runs
        for (int i = (int)threadIdx.x - 64; i < TN; i += KS_EPI_WARPS * 32) {
            const int64_t col = (int64_t)nb * TN + i;
            bias_s[i] = (p.bias != nullptr && col < p.N) ? Cvt<T>::to_f(reinterpret_cast<const T*>(p.bias)[col]) : 0.f;
        }
        bool ok = __all_sync(0xffffffffu, ptx::mbar_wait_bounded(tmem_full, 0, abort_flag));
        // All MMAs of this pair have completed: the accumulator is final and the pipeline buffers are idle.
        if (ok && S > 1) {
            ptx::tc_fence_after();
            // ---- hand the chunks that other pairs finish to their owners, straight from registers (16 bytes per
            //      message, counted on the owner's mbarrier). Work unit: 16 columns of this warp's 32 rows. ----
            const int n_units = 2 * (nch - mine);
#pragma unroll 1
            for (int u = grp; u < n_units; u += GROUPS) {
                const int j = u >> 1, half = u & 1;
                const int c = j < my_lo ? j : j + mine;
                int o = 0;
                while (chunk_lo(o + 1, S, nch) <= c) ++o;  // the pair that finishes chunk c
                const int lo = chunk_lo(o, S, nch), n_o = chunk_lo(o + 1, S, nch) - lo;
                const int sender = s < o ? s : s - 1;      // this pair's slot among the owner's S - 1 senders
                const uint32_t peer = (uint32_t)(2 * o) + r;
                uint32_t v[16];
                ptx::tmem_ld_32x16(tmem_base + lane_field + (uint32_t)(c * 32 + half * 16), v);
                ptx::tmem_ld_wait();
                const uint32_t d = ptx::map_to_cta(recv_row + (uint32_t)((sender * n_o + (c - lo)) * KS_CHUNK_BYTES + half * 4 * (BM * 16)), peer);
                const uint32_t pb = ptx::map_to_cta(ptx::smem_u32(recv_full), peer);
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    st_async_v4(d + (uint32_t)(q * (BM * 16)), v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3], pb);
            }
        }
        epilogue_bar_sync();  // reached by every epilogue thread, whatever `ok` says (also publishes bias_s)
        __syncwarp();
        // ---- finish the chunks this pair owns ----
        if (ok && S > 1) ok = __all_sync(0xffffffffu, ptx::mbar_wait_bounded(recv_full, 0, abort_flag));
        if (ok) {
            ptx::tc_fence_after();
            // unit u = 16 columns: chunk u >> 1 of this pair's share, half u & 1
            auto unit_col0 = [&](int u) { return (int64_t)nb * TN + (my_lo + (u >> 1)) * 32 + (u & 1) * 16; };
            auto unit_taddr = [&](int u) { return tmem_base + lane_field + (uint32_t)((my_lo + (u >> 1)) * 32 + (u & 1) * 16); };
            auto finish_unit = [&](int u, const uint32_t (&own)[16]) {
                const int cl = u >> 1, half = u & 1;
                float v[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) v[e] = 0.f;
                // partial sums are added in split order whichever pair does the adding
                for (int i = 0; i < S; ++i) {
                    if (i == s) {
#pragma unroll
                        for (int e = 0; e < 16; ++e) v[e] += __uint_as_float(own[e]);
                    } else {
                        const int sender = i < s ? i : i - 1;
                        const uint32_t src = recv_row + (uint32_t)((sender * mine + cl) * KS_CHUNK_BYTES + half * 4 * (BM * 16));
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const uint4 w4 = ptx::ld_shared_v4(src + (uint32_t)(q * (BM * 16)));
                            v[4 * q] += __uint_as_float(w4.x);
                            v[4 * q + 1] += __uint_as_float(w4.y);
                            v[4 * q + 2] += __uint_as_float(w4.z);
                            v[4 * q + 3] += __uint_as_float(w4.w);
                        }
                    }
                }
                store_cols16<T>(p, v, bias_s + (my_lo + cl) * 32 + half * 16, row, row < p.M, unit_col0(u));
            };
            // two units per round: both accumulator reads are in flight before either is used (a round is mostly the
            // latency of the TMEM read and of the stores, so a warp with three units to finish pays for two rounds, not three)
#pragma unroll 1
            for (int u = grp; u < 2 * mine; u += 2 * GROUPS) {
                if (unit_col0(u) >= p.N) break;  // warp-uniform; later units of this warp lie further right
                const int u2 = u + GROUPS;
                const bool second = u2 < 2 * mine && unit_col0(u2) < p.N;
                uint32_t own[16], own2[16];
                ptx::tmem_ld_32x16(unit_taddr(u), own);
                if (second) ptx::tmem_ld_32x16(unit_taddr(u2), own2);
                ptx::tmem_ld_wait();
                finish_unit(u, own);
                if (second) finish_unit(u2, own2);
            }
        }
        if (!ok && lane == 0) atomicOr(&g_ksplit_status[0], 4u);
    }

    // ------------------------------ teardown --------------------------------------
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();  // no CTA leaves (or frees TMEM) while a peer may still write to it or signal it
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, TILE);
    }
}

// How many clusters of 2*S CTAs of this kernel can be resident at once (cached per S and kernel instantiation).
template <typename T>
int max_active_clusters(int S) {
    static thread_local int cached[KS_MAX_SPLIT + 1] = {0, 0, 0, 0, 0};
    if (cached[S] > 0) return cached[S];
    auto kern = gemm_tc_ksplit_kernel<T>;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * S * 64));
    cfg.blockDim = dim3(KS_THREADS);
    cfg.dynamicSmemBytes = KS_SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = (unsigned)(2 * S);
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        static const int on_b200[KS_MAX_SPLIT + 1] = {0, 74, 33, 22, 15};  // what a 148-SM B200 reports
        n = on_b200[S] * num_sms() / 148;
        if (n < 1) n = 1;
    }
    cached[S] = n;
    return n;
}

template <typename T>
int launch_ksplit(const void* A, const void* W, const void* bias, const void* residual, void* out, int64_t M, int64_t N,
                  int64_t K, int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int act, int S, int tn, cudaStream_t st) {
    constexpr bool is_bf16 = std::is_same<T, __nv_bfloat16>::value;
    auto kern = gemm_tc_ksplit_kernel<T>;
    static thread_local bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, KS_SMEM_BYTES);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(XG_ERR_LAUNCH, "xg_gemm_bias_act: cannot reserve %d bytes of shared memory: %s", KS_SMEM_BYTES,
                        cudaGetErrorString(e));
        }
        attr_set = true;
    }
    CUtensorMap ta, tw;
    if (!make_tmap_2d_16bit(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM, BK, is_bf16) ||
        !make_tmap_2d_16bit(&tw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, (uint32_t)(tn / 2), BK, is_bf16))
        return fail(XG_ERR_UNSUPPORTED, "xg_gemm_bias_act: tensor-map encoding failed (M=%lld N=%lld K=%lld lda=%lld ldb=%lld)",
                    (long long)M, (long long)N, (long long)K, (long long)lda, (long long)ldw);
    KsplitParams p;
    p.out = out;
    p.bias = bias;
    p.residual = residual;
    p.M = M; p.N = N; p.ldc = ldc; p.ldr = ldr;
    p.act = act;
    p.vec_ok = (ldc % 8 == 0) && aligned16(out) && (!residual || (ldr % 8 == 0 && aligned16(residual)));
    p.bias_vec_ok = bias ? aligned16(bias) : 0;
    p.num_m_blocks = (int)((M + TILE - 1) / TILE);
    p.num_n_blocks = (int)((N + tn - 1) / tn);
    p.num_k_blocks = (int)((K + BK - 1) / BK);
    p.S = S;
    p.tn = tn;
    p.stages = S > 1 ? KS_STAGES_SPLIT : KS_STAGES_WHOLE;
    const int64_t tiles = (int64_t)p.num_m_blocks * p.num_n_blocks;
    if (tiles * 2 * S > 0x7fffffffLL) return fail(XG_ERR_TOO_LARGE, "xg_gemm_bias_act: too many tiles for one launch");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles * 2 * S));
    cfg.blockDim = dim3(KS_THREADS);
    cfg.dynamicSmemBytes = KS_SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = (unsigned)(2 * S);
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaError_t le = cudaLaunchKernelEx(&cfg, kern, ta, tw, p);
    if (le != cudaSuccess) {
        cudaGetLastError();
        return fail(XG_ERR_LAUNCH, "xg_gemm_bias_act (k-split clusters of %d): %s", 2 * S, cudaGetErrorString(le));
    }
    return XG_OK;
}

bool ksplit_shape_ok(int S, int tn, int64_t nkb) {
    return S >= 1 && S <= KS_MAX_SPLIT && tn >= 64 && tn <= TILE && tn % 32 == 0 && tn / 32 >= S && nkb >= S;
}

}  // namespace

// Whether the cluster kernel should run an [M, N, K] problem (W given as [N, K]) and how: the number of k-splits S (1..4)
// and the tile width tn; returns false when another kernel is the better choice. XG_GEMM_KSPLIT="S" or "S,tn"
// overrides the choice (S = 0: never).
//
// The choice rests on a cost model in microseconds fitted to measurements on B200 (K = 4096, M = 16..1024,
// N = 520..11008, every (S, tn) below): a CTA of a pair takes in its 16 KiB of activations and tn/2 weight rows per
// k-block in about 0.0142 us per KiB - 0.124 us (20..32 KiB; the tensor time of the k-block, tn/256 * 0.26 us, is
// the floor); a wave of clusters costs about 3.6 us to set up, drain and launch; the finishing pass takes 0.9 us per
// round of four 16-column units per lane quadrant; a split adds the staging pass (0.35 us per round), the exchange at
// about 45 KB/us per CTA and 0.5 us of synchronisation. The alternative - independent 128-row CTAs - streams at
// about 127 KB/us per SM plus 3 us. The cluster kernel runs when it comes out at least 10 % ahead, which for
// K = 4096 means 128 < M <= 512 at N = 4096 (13.3 vs 15.7 us at M = 256, 19.6 vs 26.9 us at M = 512) and M <= 256 at
// N = 11008 (22.3 vs 36.3 us), and shapes with between one and two waves of 256 x 256 tiles (512 x 11008: 43 vs
// 51 us for the pair kernel). Smaller M stays with split-K through scratch, which is ahead there.
bool plan_ksplit(int64_t M, int64_t N, int64_t K, int dtype, int* S_out, int* tn_out) {
    static const int forced_s = []() {
        const char* e = getenv("XG_GEMM_KSPLIT");
        return e ? atoi(e) : -1;
    }();
    static const int forced_tn = []() {
        const char* e = getenv("XG_GEMM_KSPLIT");
        const char* c = e ? strchr(e, ',') : nullptr;
        return c ? atoi(c + 1) : TILE;
    }();
    const int64_t nkb = (K + BK - 1) / BK;
    const int64_t mblk = (M + TILE - 1) / TILE;
    if (forced_s == 0 || M <= 0 || N <= 0) return false;
    if (forced_s > 0) {
        if (!ksplit_shape_ok(forced_s, forced_tn, nkb) || mblk * ((N + forced_tn - 1) / forced_tn) > 0x7fffff) return false;
        *S_out = forced_s;
        *tn_out = forced_tn;
        return true;
    }
    if (M <= 128 || nkb < 8) return false;  // small M: split-K through scratch is ahead; short K: nothing to stream
    const int sms = num_sms();
    const int64_t tiles256 = mblk * ((N + 255) / 256);
    if (tiles256 >= sms) return false;  // two full waves or more of 256 x 256 tiles: the persistent pair kernel's regime
    auto per_kblock = [](double kib, int tn) {
        const double load = 0.0142 * kib - 0.124, mma = tn / 256.0 * 0.26;
        const double t = load > mma ? load : mma;
        return t > 0.12 ? t : 0.12;
    };
    auto rounds = [](int chunks) { return (double)((2 * chunks + KS_EPI_WARPS / 4 - 1) / (KS_EPI_WARPS / 4)); };
    double best = 1e30;
    int best_s = 0, best_tn = 0;
    for (int tn = 64; tn <= TILE; tn += 32) {
        const int64_t tiles = mblk * ((N + tn - 1) / tn);
        const int nch = tn / 32;
        for (int S = 1; S <= KS_MAX_SPLIT; ++S) {
            if (!ksplit_shape_ok(S, tn, nkb) || (S > 1 && nkb < 8 * S)) continue;
            const int active = dtype == XG_BF16 ? max_active_clusters<__nv_bfloat16>(S) : max_active_clusters<__half>(S);
            const double waves = (double)((tiles + active - 1) / active);
            const int own = (nch + S - 1) / S, sent = nch - nch / S;
            double wave = (double)((nkb + S - 1) / S) * per_kblock(16.0 + tn / 2 * 0.125, tn) + 3.6 + 0.9 * rounds(own);
            if (S > 1) wave += 0.35 * rounds(sent) + sent * 16.0 / 45.0 + 0.5;
            const double cost = waves * wave;
            if (cost < best) { best = cost; best_s = S; best_tn = tn; }
        }
    }
    if (best_s == 0) return false;
    // the alternative: 128-row CTAs with the widest tile that still gives every SM work
    const int64_t mblk128 = (M + BM - 1) / BM;
    int bn = 256;
    if (mblk128 * ((N + 255) / 256) < sms) bn = 128;
    if (bn == 128 && mblk128 * ((N + 127) / 128) < sms) bn = 64;
    const int64_t ctas = mblk128 * ((N + bn - 1) / bn);
    double other = (double)((ctas + sms - 1) / sms) * (double)nkb * (16.0 + bn * 0.125) / 127.0 + 3.0;
    if (tiles256 >= sms / 2) {
        // between one and two waves of 256 x 256 tiles the dispatcher would take the persistent pair kernel, whose last
        // wave is mostly empty (86 tiles on 74 pairs: 51 us at 512 x 4096 x 11008 against 43 us for 138 tiles of 160 columns)
        const double pair = (double)((tiles256 + sms / 2 - 1) / (sms / 2)) * ((double)nkb * per_kblock(32.0, 256) + 3.6);
        if (pair < other) other = pair;
    }
    if (best > 0.9 * other) return false;
    *S_out = best_s;
    *tn_out = best_tn;
    return true;
}

int gemm_tc_ksplit_entry(const void* A, const void* W, const void* bias, const void* residual, void* out, int64_t M,
                         int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldc, int64_t ldr, int act, int dtype, int S,
                         int tn, cudaStream_t st) {
    if (!ksplit_shape_ok(S, tn, (K + BK - 1) / BK))
        return fail(XG_ERR_INVALID_ARG, "xg_gemm_bias_act: bad k-split %d / tile width %d", S, tn);
    if (dtype == XG_BF16)
        return launch_ksplit<__nv_bfloat16>(A, W, bias, residual, out, M, N, K, lda, ldw, ldc, ldr, act, S, tn, st);
    return launch_ksplit<__half>(A, W, bias, residual, out, M, N, K, lda, ldw, ldc, ldr, act, S, tn, st);
}

int read_ksplit_status(unsigned int* host_out, int reset) {
    unsigned int v[4] = {0, 0, 0, 0};
    if (cudaMemcpyFromSymbol(v, g_ksplit_status, sizeof(v)) != cudaSuccess) {
        cudaGetLastError();
        return fail(XG_ERR_DEVICE, "xg_tc_status: cannot read device status");
    }
    *host_out = v[0];
    if (reset && v[0] != 0) {
        unsigned int z[4] = {0, 0, 0, 0};
        cudaMemcpyToSymbol(g_ksplit_status, z, sizeof(z));
    }
    return XG_OK;
}

}  // namespace xg
