// Fused scaled-dot-product attention: out = softmax(q k^T * scale + mask) v, online softmax.
//
// 16-bit inputs with head_dim 64 or 128 run on the tensor cores (flash_tc_kernel):
//   one CTA per (batch, head, 128-query tile); warp 0 streams K/V tiles with TMA (2-stage ring),
//   warp 1's elected thread issues tcgen05.mma for S = Q K^T (into one of two TMEM buffers, so the
//   next block's scores are computed while the current block is in softmax) and for P V (P read from
//   TMEM, V consumed MN-major exactly as TMA leaves it); warps 2..5 own one query row per thread: they
//   read the row's scores from TMEM, keep the running max / sum and write the probabilities back as
//   packed 16-bit pairs over the first half of the same score buffer, so a block's softmax never waits
//   for the previous block's P V. O accumulates in TMEM and is rescaled lazily.
//   Causal tiles beyond the diagonal are skipped.
// Everything else runs in true fp32 on SIMT kernels: a shared-memory tiled kernel (head dim 32 / 64 / 128, no additive
// mask) and a warp-per-query kernel (masks, other head dims).
#include "common.cuh"
#include "sm100_ptx.cuh"

#include <type_traits>

namespace xg {

// Status word of the attention kernel (device globals are per translation unit without -rdc).
__device__ unsigned int g_sdpa_status[4];

namespace {

constexpr float kLog2e = 1.4426950408889634f;

struct SdpaParams {
    const void* q;
    const void* k;
    const void* v;
    const void* mask;
    void* out;
    int64_t B, H, Sq, Skv, D;
    int64_t q_sb, q_sh, q_ss;
    int64_t k_sb, k_sh, k_ss;
    int64_t v_sb, v_sh, v_ss;
    int64_t o_sb, o_sh, o_ss;
    int64_t m_sb, m_sh, m_sq, m_sk;
    float scale;
    int causal;
};

// ---------------------------------------------------------------------------------------
// Tensor-core flash kernel
// ---------------------------------------------------------------------------------------
// What the tensor-core kernel needs beside its three tensor maps (which carry q, k, v and their strides), kept under
// 128 bytes so that the kernel's parameter block stays within 512 bytes (a larger block was measured to slow the GEMM
// kernels of this library down by up to 30 %).
struct FlashParams {
    const void* mask;
    void* out;
    int64_t o_sb, o_sh, o_ss;
    int64_t m_sb, m_sh, m_sq, m_sk;
    int B, H, Sq, Skv;
    float scale;
    int causal;
};
static_assert(sizeof(FlashParams) <= 128, "flash kernel parameter block must stay within 512 bytes");

constexpr int FM = 128;  // query rows per CTA
constexpr int FN = 64;   // keys per block
constexpr int kFlashThreads = 192;
constexpr float kRescaleThreshold = 8.0f;  // log2 units: the running max may lag by up to 2^8

template <int D>
struct FlashCfg {
    static constexpr int DB = D / 64;                 // 64-wide head-dim blocks
    static constexpr int Q_BYTES = FM * D * 2;
    static constexpr int KV_BYTES = FN * D * 2;       // one K or V tile
    // Two CTAs share an SM, and the window carries no alignment slack: the kernel checks that the
    // dynamic shared-memory window starts on a 1024-byte boundary and reports if it does not.
    static constexpr int O_STAGE_BYTES = 4 * 32 * 128;  // a 32-row, 64-column slab per softmax warp
    static constexpr int SMEM_BYTES = Q_BYTES + 4 * KV_BYTES + O_STAGE_BYTES + 256;  // tiles + staging + barriers
    static_assert(2 * (SMEM_BYTES + 1024) <= 233472, "two CTAs must fit in one SM's shared memory");
    // S0 [0,64) S1 [64,128) O [128, 128+D); P of block n overlays columns [0,32) of score buffer n & 1
    static constexpr int TMEM_COLS = 256;
    static constexpr uint32_t O_COL = 128;
};

// Work list of the persistent CTAs: tile L -> (batch*head, query tile). Consecutive L stay inside one
// (batch, head), so the CTAs running at the same time share that head's K/V through L2. Within a head the
// causal order alternates heavy and light query tiles (last, first, last-1, second, ...): any two neighbours
// add up to the same number of key blocks, so a CTA that takes every gridDim.x-th tile gets an even share
// (the host makes gridDim.x even).
struct FlashTile {
    int b, h, q0, nblk;
};
__device__ __forceinline__ FlashTile flash_tile(const FlashParams& p, int b, int h, int k, int q_tiles) {
    const int qt = p.causal ? ((k & 1) ? (k >> 1) : (q_tiles - 1 - (k >> 1))) : k;
    FlashTile t;
    t.h = h;
    t.b = b;
    t.q0 = qt * FM;
    t.nblk = (int)((p.Skv + FN - 1) / FN);
    if (p.causal) {
        const int lim = (t.q0 + FM - 1) / FN + 1;  // last block that any row of this tile can see
        if (lim < t.nblk) t.nblk = lim;
    }
    return t;
}

// A CTA takes neighbouring tiles in pairs (2c, 2c+1), then (2(c+G), 2(c+G)+1), ... Every role walks that list with
// a cursor that keeps (batch, head, position in the head) of the pair's first tile and adds the decoded stride, so
// that the integer divisions happen once per kernel and not once per tile.
struct FlashCursor {
    int L;        // list index of the current pair's first tile
    int b, h, k;  // its batch, head and position in the head's order
};
struct FlashStride {  // 2 * gridDim.x tiles, decoded the same way (kept in shared memory)
    int db, dh, dk;
};
__device__ __forceinline__ void flash_carry(int& b, int& h, int& k, int q_tiles, int H) {
    if (k >= q_tiles) { k -= q_tiles; ++h; }
    if (h >= H) { h -= H; ++b; }
}
__device__ __forceinline__ FlashStride flash_stride(const FlashParams& p, int q_tiles) {
    FlashStride s;
    const int step = 2 * (int)gridDim.x;
    const int bh = step / q_tiles;
    s.dk = step - bh * q_tiles;
    s.db = bh / p.H;
    s.dh = bh - s.db * p.H;
    return s;
}
__device__ __forceinline__ FlashCursor flash_cursor(const FlashParams& p, int q_tiles) {
    FlashCursor c;
    c.L = 2 * (int)blockIdx.x;
    const int bh = c.L / q_tiles;
    c.k = c.L - bh * q_tiles;
    c.b = bh / p.H;
    c.h = bh - c.b * p.H;
    return c;
}
// i-th tile of this CTA (i = 0, 1, 2, ... in order). Returns 0 with the tile in t, -1 when the CTA is done, -2 for
// the missing second half of a trailing odd pair.
__device__ __forceinline__ int flash_next(FlashCursor& c, const volatile FlashStride* stride, int i, int num_tiles, int q_tiles,
                                          const FlashParams& p, FlashTile& t) {
    if ((i & 1) == 0) {
        if (i > 0) {
            c.L += 2 * (int)gridDim.x;
            c.k += stride->dk;
            c.h += stride->dh;
            c.b += stride->db;
            flash_carry(c.b, c.h, c.k, q_tiles, p.H);  // k < 2 q_tiles and h <= 2 H - 1 here: one carry each is enough
        }
        if (c.L >= num_tiles) return -1;
        t = flash_tile(p, c.b, c.h, c.k, q_tiles);
        return 0;
    }
    if (c.L + 1 >= num_tiles) return -2;
    int b = c.b, h = c.h, k = c.k + 1;
    flash_carry(b, h, k, q_tiles, p.H);
    t = flash_tile(p, b, h, k, q_tiles);
    return 0;
}

// MASKED: the kernel carries the general masking code (additive mask, key count that is not a multiple of the block,
// non-positive scale). The common case is compiled without it: the code of a tile boundary runs once per tile, its
// instruction fetches miss the instruction caches, and a smaller kernel keeps more of it resident.
template <typename T, int D, bool MASKED>
__global__ void __launch_bounds__(kFlashThreads, 2)
flash_tc_kernel(const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmk,
                const __grid_constant__ CUtensorMap tmv, const FlashParams p) {
    using Cfg = FlashCfg<D>;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* q_s = smem;
    uint8_t* k_s = q_s + Cfg::Q_BYTES;            // [2][KV_BYTES]
    uint8_t* v_s = k_s + 2 * Cfg::KV_BYTES;       // [2][KV_BYTES]
    uint8_t* o_stage = v_s + 2 * Cfg::KV_BYTES;   // [4 warps][32 rows][128 bytes]: output rows on their way out
    uint64_t* bars = reinterpret_cast<uint64_t*>(o_stage + Cfg::O_STAGE_BYTES);
    uint64_t* q_full = bars;          // 1   one phase per tile
    uint64_t* k_full = bars + 1;      // 2   the block barriers below run on per-role block counters that
    uint64_t* k_empty = bars + 3;     // 2   keep counting across the tiles of this CTA
    uint64_t* v_full = bars + 5;      // 2
    uint64_t* v_empty = bars + 7;     // 2
    uint64_t* s_full = bars + 9;      // 2
    uint64_t* o_full = bars + 11;     // 1   one phase per tile: the tile's last P V has completed
    uint64_t* p_full = bars + 12;     // 2   a softmax warp may run one block ahead of the slowest one
    uint64_t* pv_full = bars + 14;    // 1
    uint64_t* drain_bar = bars + 15;  // 1
    uint64_t* q_empty = bars + 16;    // 1   all Q K^T of a tile have read Q
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile FlashStride* stride = reinterpret_cast<volatile FlashStride*>(tmem_slot + 2);

    if ((ptx::smem_u32(smem) & 1023u) != 0) {  // uniform over the CTA: the swizzled tiles need this alignment
        if (threadIdx.x == 0) atomicOr(&g_sdpa_status[0], 128u);
        return;
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_tiles = (int)((p.Sq + FM - 1) / FM);
    const int num_tiles = q_tiles * (int)(p.B * p.H);

    if (threadIdx.x == 0) {
        ptx::mbar_init(q_full, 1);
        ptx::mbar_init(q_empty, 1);
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_init(&k_full[s], 1);
            ptx::mbar_init(&k_empty[s], 1);
            ptx::mbar_init(&v_full[s], 1);
            ptx::mbar_init(&v_empty[s], 1);
            ptx::mbar_init(&s_full[s], 1);
        }
        ptx::mbar_init(&p_full[0], 128);
        ptx::mbar_init(&p_full[1], 128);
        ptx::mbar_init(pv_full, 1);
        ptx::mbar_init(o_full, 1);
        ptx::mbar_init(drain_bar, 1);
        *abort_flag = 0;
        {
            const FlashStride st = flash_stride(p, q_tiles);
            stride->db = st.db;
            stride->dh = st.dh;
            stride->dk = st.dk;
        }
        ptx::fence_mbar_init();
        ptx::fence_proxy_async();
    }
    if (warp == 1) ptx::tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (ptx::elect_one()) {
            ptx::prefetch_tensormap(&tmq);
            ptx::prefetch_tensormap(&tmk);
            ptx::prefetch_tensormap(&tmv);
            bool ok = true;
            uint32_t n = 0;      // key blocks loaded so far (all tiles)
            uint32_t tile_n = 0; // tiles started so far
            FlashCursor cur = flash_cursor(p, q_tiles);
            for (int i = 0; ok; ++i) {
                FlashTile t;
                const int tile_state = flash_next(cur, stride, i, num_tiles, q_tiles, p, t);
                if (tile_state == -1) break;
                if (tile_state == -2) continue;
                const uint32_t tile_par = tile_n++ & 1u;
                // Q may be overwritten once every Q K^T of the previous tile has completed
                if (!ptx::mbar_wait_bounded(q_empty, tile_par ^ 1u, abort_flag)) { ok = false; break; }
                ptx::mbar_arrive_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
                for (int db = 0; db < Cfg::DB; ++db) ptx::tma_load_4d(q_s + db * (FM * 128), &tmq, q_full, db * 64, t.q0, t.h, t.b);
                for (int j = 0; j < t.nblk; ++j, ++n) {
                    const int s = (int)(n & 1u);
                    const uint32_t ph = (n >> 1) & 1u;
                    if (!ptx::mbar_wait_bounded(&k_empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                    ptx::mbar_arrive_expect_tx(&k_full[s], Cfg::KV_BYTES);
#pragma unroll
                    for (int db = 0; db < Cfg::DB; ++db)
                        ptx::tma_load_4d(k_s + s * Cfg::KV_BYTES + db * (FN * 128), &tmk, &k_full[s], db * 64, j * FN, t.h, t.b);
                    if (!ptx::mbar_wait_bounded(&v_empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                    ptx::mbar_arrive_expect_tx(&v_full[s], Cfg::KV_BYTES);
#pragma unroll
                    for (int db = 0; db < Cfg::DB; ++db)
                        ptx::tma_load_4d(v_s + s * Cfg::KV_BYTES + db * (FN * 128), &tmv, &v_full[s], db * 64, j * FN, t.h, t.b);
                }
            }
            if (!ok) {
                // Unwinding: give this thread's own copies a bounded time to land before shared memory is given up.
                atomicOr(&g_sdpa_status[0], 16u);
                const uint64_t t0 = ptx::globaltimer_ns();
                while (ptx::globaltimer_ns() - t0 < 20000ull) {
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (ptx::elect_one()) {
            constexpr uint32_t idesc_s = ptx::make_idesc_f16(fmt, FM, FN, 0);
            constexpr uint32_t idesc_o = ptx::make_idesc_f16(fmt, FM, D, 1);
            const uint32_t q_addr = ptx::smem_u32(q_s);
            bool ok = true;
            uint32_t nq = 0;  // Q K^T blocks issued so far (all tiles)
            uint32_t np = 0;  // P V blocks issued so far
            uint32_t tile_n = 0;
            FlashCursor cur = flash_cursor(p, q_tiles);
            // Score buffer nq & 1 is free without a barrier of its own: this thread has already waited for
            // p_full of block nq - 2 (the softmax warps had read S and written P by then) and issued that
            // block's P V before this point, and the tensor core runs this thread's MMAs in issue order.
            auto issue_qk = [&]() -> bool {
                const int s = (int)(nq & 1u);
                const uint32_t ph = (nq >> 1) & 1u;
                if (!ptx::mbar_wait_bounded(&k_full[s], ph, abort_flag)) return false;
                ptx::tc_fence_after();
                const uint32_t k_addr = ptx::smem_u32(k_s + s * Cfg::KV_BYTES);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t q_off = (uint32_t)((kk >> 2) * (FM * 128) + (kk & 3) * 32);
                    const uint32_t k_off = (uint32_t)((kk >> 2) * (FN * 128) + (kk & 3) * 32);
                    ptx::mma_f16_ss(tmem_base + (uint32_t)(s * FN), ptx::make_kmajor_sw128_desc(q_addr + q_off),
                                    ptx::make_kmajor_sw128_desc(k_addr + k_off), idesc_s, kk != 0 ? 1u : 0u);
                }
                ptx::tc_commit(&k_empty[s]);
                ptx::tc_commit(&s_full[s]);
                ++nq;
                return true;
            };
            for (int i = 0; ok; ++i) {
                FlashTile t;
                const int tile_state = flash_next(cur, stride, i, num_tiles, q_tiles, p, t);
                if (tile_state == -1) break;
                if (tile_state == -2) continue;
                if (!ptx::mbar_wait_bounded(q_full, tile_n++ & 1u, abort_flag)) { ok = false; break; }
                if (t.nblk > 0) ok = issue_qk();
                if (ok && t.nblk == 1) ptx::tc_commit(q_empty);
                for (int j = 0; j < t.nblk && ok; ++j, ++np) {
                    if (j + 1 < t.nblk) {
                        if (!issue_qk()) { ok = false; break; }
                        if (j + 2 == t.nblk) ptx::tc_commit(q_empty);  // that was the tile's last Q K^T
                    }
                    const int s = (int)(np & 1u);
                    if (!ptx::mbar_wait_bounded(&p_full[s], (np >> 1) & 1u, abort_flag)) { ok = false; break; }
                    if (!ptx::mbar_wait_bounded(&v_full[s], (np >> 1) & 1u, abort_flag)) { ok = false; break; }
                    ptx::tc_fence_after();
                    const uint32_t v_addr = ptx::smem_u32(v_s + s * Cfg::KV_BYTES);
#pragma unroll
                    for (int kk = 0; kk < FN / 16; ++kk) {
                        // O (+)= P V: the tile's first block overwrites, later blocks accumulate in TMEM
                        // P: 16 keys = 8 TMEM columns of packed pairs per step, in score buffer np & 1
                        ptx::mma_f16_ts(tmem_base + Cfg::O_COL, tmem_base + (uint32_t)(s * FN + kk * 8),
                                        ptx::make_mnmajor_sw128_desc(v_addr + (uint32_t)(kk * 16 * 128), FN * 128), idesc_o,
                                        (j | kk) != 0 ? 1u : 0u);
                    }
                    ptx::tc_commit(&v_empty[s]);
                    ptx::tc_commit(pv_full);
                    if (j + 1 == t.nblk) ptx::tc_commit(o_full);
                }
                if (ok && t.nblk == 0) ptx::tc_commit(q_empty);
            }
            if (!ok) {
                atomicOr(&g_sdpa_status[0], 32u);
                ptx::tc_commit(drain_bar);
                const uint64_t t0 = ptx::globaltimer_ns();
                while (!ptx::mbar_try_wait(drain_bar, 0)) {
                    if (ptx::globaltimer_ns() - t0 > ptx::kWaitLimitNs) break;
                }
            }
        }
    } else {
        // ------------------------------ softmax / output rows ---------------------
        // One query row per thread. The output accumulates in TMEM; it is rescaled only when some row
        // of the warp sees its maximum grow by more than 2^kRescaleThreshold (the running maximum is
        // allowed to lag, the final division by the row sum makes the result exact either way).
        const int quad = warp & 3;
        const int r_in_tile = quad * 32 + lane;
        const uint32_t lane_field = (uint32_t)(quad * 32) << 16;
        const float sl2 = p.scale * kLog2e;
        const int skv = (int)p.Skv;
        bool ok = true;
        uint32_t n = 0;       // key blocks processed so far (all tiles)
        uint32_t tile_n = 0;  // tiles finished so far
        FlashCursor cur = flash_cursor(p, q_tiles);

        for (int i = 0; ok; ++i) {
            FlashTile t;
            const int tile_state = flash_next(cur, stride, i, num_tiles, q_tiles, p, t);
            if (tile_state == -1) break;
            if (tile_state == -2) continue;
            const int q0 = t.q0, nblk = t.nblk;
            const int row = q0 + r_in_tile;
            const T* mrow = nullptr;
            if (MASKED && p.mask != nullptr && row < p.Sq)
                mrow = reinterpret_cast<const T*>(p.mask) + (int64_t)t.b * p.m_sb + (int64_t)t.h * p.m_sh + (int64_t)row * p.m_sq;
            float m_run = -INFINITY, l_run = 0.f;  // running maximum (log2 domain, scaled) and row sum

            for (int j = 0; j < nblk; ++j, ++n) {
                const int sb = (int)(n & 1u);
                // wait results are made warp-uniform: the TMEM accesses below are warp-collective
                if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(&s_full[sb], (n >> 1) & 1u, abort_flag))) { ok = false; break; }
                ptx::tc_fence_after();
                const uint32_t s_taddr = tmem_base + lane_field + (uint32_t)(sb * FN);
                const int col_base = j * FN;
                // A block needs the general masking code when it carries an additive mask, crosses the end of the
                // keys or has a non-positive scale. A block that is only cut by the causal diagonal is classified per
                // warp (a warp owns 32 consecutive query rows): all keys visible, some, or none.
                const bool general_mask = MASKED && ((p.mask != nullptr) || (col_base + FN > skv) || !(sl2 > 0.f));
                const int warp_row0 = q0 + quad * 32;
                const bool diag_none = !general_mask && p.causal && (col_base > warp_row0 + 31);
                const bool diag_some = !general_mask && p.causal && !diag_none && (col_base + FN - 1 > warp_row0);
                if (diag_none) {
                    // every key of the block lies beyond the diagonal for these rows: the probabilities are zero and
                    // neither the running maximum nor the row sum moves
                    uint32_t zero[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) zero[i] = 0u;
                    ptx::tmem_st_32x32(s_taddr, zero);
                    ptx::tmem_st_wait();
                    ptx::tc_fence_before();
                    ptx::mbar_arrive(&p_full[sb]);
                    continue;
                }
                float sc[FN];  // raw scores; exp2(sc * mul - m) is the probability
                {
                    uint32_t r0[32], r1[32];
                    ptx::tmem_ld_32x32(s_taddr, r0);
                    ptx::tmem_ld_32x32(s_taddr + 32u, r1);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        sc[i] = __uint_as_float(r0[i]);
                        sc[32 + i] = __uint_as_float(r1[i]);
                    }
                }
                float mul = sl2;
                if (diag_some) {  // raw scores beyond the diagonal become -inf; the scale stays in the exponent's FMA
                    const int last_visible = row - col_base;
#pragma unroll
                    for (int i = 0; i < FN; ++i)
                        if (i > last_visible) sc[i] = -INFINITY;
                }
                if (MASKED && general_mask) {  // uniform over the CTA; scores go to the log2 domain here
#pragma unroll
                    for (int i = 0; i < FN; ++i) {
                        const int col = col_base + i;
                        sc[i] *= sl2;
                        if (mrow != nullptr && col < skv) sc[i] += Cvt<T>::to_f(mrow[(int64_t)col * p.m_sk]) * kLog2e;
                        if (col >= skv || (p.causal && col > row)) sc[i] = -INFINITY;
                    }
                    mul = 1.f;
                }
                // The first block of a tile needs its maximum before any probability can be formed. Later blocks form
                // their probabilities against the running maximum at once, while the block's own maximum is reduced
                // alongside (the two instruction streams are independent); only when some row's maximum grew beyond the
                // threshold - rare after a tile's first blocks - is O rescaled and the block done again.
                if (j == 0) {
                    // 8 independent chains of 3-input maxima instead of one 64-deep dependency chain
                    float mxp[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) mxp[i] = ptx::fmax3(sc[i], sc[8 + i], sc[16 + i]);
#pragma unroll
                    for (int i = 24; i < FN; i += 16)
#pragma unroll
                        for (int c = 0; c < 8; ++c) mxp[c] = ptx::fmax3(mxp[c], sc[i + c], sc[i + 8 + c]);
                    // (i = 24: 24..39, i = 40: 40..55) leaves 56..63
#pragma unroll
                    for (int c = 0; c < 8; ++c) mxp[c] = fmaxf(mxp[c], sc[56 + c]);
                    m_run = ptx::fmax3(ptx::fmax3(mxp[0], mxp[1], mxp[2]), ptx::fmax3(mxp[3], mxp[4], mxp[5]),
                                       fmaxf(mxp[6], mxp[7])) * mul;
                }
                // probabilities -> packed 16-bit pairs over columns [0, 32) of this block's score buffer
                uint32_t pk[32];
#pragma unroll 1
                for (int attempt = 0; attempt < 2; ++attempt) {
                    const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
                    float lp[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};  // independent partial row sums (4 pairs)
                    float mxp[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) mxp[i] = -INFINITY;
#pragma unroll
                    for (int i = 0; i < FN; i += 2) {
                        float x0, x1, p0, p1;
                        ptx::fma2(x0, x1, sc[i], sc[i + 1], mul, mul, neg_m, neg_m);
                        const int pair = i >> 1;
                        p0 = ptx::ex2_approx(x0);
                        p1 = ptx::ex2_approx(x1);
                        mxp[pair & 7] = ptx::fmax3(mxp[pair & 7], sc[i], sc[i + 1]);
                        ptx::add2(lp[2 * (pair & 3)], lp[2 * (pair & 3) + 1], lp[2 * (pair & 3)], lp[2 * (pair & 3) + 1], p0, p1);
                        pk[pair] = ptx::pack2<T>(p0, p1);
                    }
                    const float l_blk = ((lp[0] + lp[1]) + (lp[2] + lp[3])) + ((lp[4] + lp[5]) + (lp[6] + lp[7]));
                    if (attempt == 0 && j > 0) {  // uniform over the CTA
                        const float mx = ptx::fmax3(ptx::fmax3(mxp[0], mxp[1], mxp[2]), ptx::fmax3(mxp[3], mxp[4], mxp[5]),
                                                    fmaxf(mxp[6], mxp[7])) * mul;
                        const float m_new = fmaxf(m_run, mx);
                        const bool grow = m_new > m_run + kRescaleThreshold;  // also true for the first finite maximum
                        if (__any_sync(0xffffffffu, grow)) {
                            const float m_to = (m_new == -INFINITY) ? 0.f : m_new;
                            const float alpha = ptx::ex2_approx(m_run - m_to);  // 0 when there was no finite maximum yet
                            // O must be quiescent: P V of the previous block has completed. s_full of this block
                            // already implies the P V two blocks back, so the barrier is at most one phase behind.
                            if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(pv_full, (n - 1) & 1u, abort_flag))) { ok = false; break; }
                            ptx::tc_fence_after();
#pragma unroll 1
                            for (int c = 0; c < D / 32; ++c) {  // rare path: kept small
                                uint32_t o[32];
                                const uint32_t o_taddr = tmem_base + lane_field + Cfg::O_COL + (uint32_t)(c * 32);
                                ptx::tmem_ld_32x32(o_taddr, o);
                                ptx::tmem_ld_wait();
#pragma unroll
                                for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                                ptx::tmem_st_32x32(o_taddr, o);
                            }
                            l_run *= alpha;
                            m_run = m_new;
                            continue;  // once more, against the new maximum
                        }
                    }
                    l_run += l_blk;
                    break;
                }
                if (!ok) break;
                ptx::tmem_st_32x32(s_taddr, pk);
                ptx::tmem_st_wait();  // P (and a rescaled O) are in TMEM before the P V is released
                ptx::tc_fence_before();
                ptx::mbar_arrive(&p_full[sb]);
            }
            if (!ok) break;
            if (nblk > 0) {
                if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(o_full, tile_n & 1u, abort_flag))) { ok = false; break; }
                ++tile_n;
            }
            ptx::tc_fence_after();
            const float inv_l = 1.0f / l_run;
            // A thread holds one output row, so storing from registers would touch 32 different lines per
            // instruction. The rows go through a 4 KiB slab of shared memory per warp instead (64 head-dim columns
            // at a time, 16-byte pieces XOR-swizzled by row so that neither side has bank conflicts) and leave as
            // full 128-byte row segments, four rows per store instruction.
            T* obase = reinterpret_cast<T*>(p.out) + (int64_t)t.b * p.o_sb + (int64_t)t.h * p.o_sh;
            const uint32_t slab = ptx::smem_u32(o_stage) + (uint32_t)(quad * 4096);
            // (not unrolled: this code runs once per tile, and its instruction fetches are what it costs)
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                uint32_t o[32];
                if (nblk > 0) {
                    ptx::tmem_ld_32x32(tmem_base + lane_field + Cfg::O_COL + (uint32_t)(c * 32), o);
                    ptx::tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = 0u;
                }
#pragma unroll
                for (int t4 = 0; t4 < 4; ++t4) {
                    uint32_t w[4];  // eight outputs as packed 16-bit pairs
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float x0, x1;
                        ptx::fma2(x0, x1, __uint_as_float(o[t4 * 8 + 2 * i]), __uint_as_float(o[t4 * 8 + 2 * i + 1]), inv_l, inv_l, 0.f, 0.f);
                        w[i] = ptx::pack2<T>(x0, x1);
                    }
                    const int piece = (c & 1) * 4 + t4;  // 16-byte piece of this row's 128-byte segment
                    ptx::st_shared_v4(slab + (uint32_t)(lane * 128 + ((piece ^ (lane & 7)) << 4)), make_uint4(w[0], w[1], w[2], w[3]));
                }
                if (c & 1) {
                    __syncwarp();
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int r = it * 4 + (lane >> 3), piece = lane & 7;
                        const uint4 val = ptx::ld_shared_v4(slab + (uint32_t)(r * 128 + ((piece ^ (r & 7)) << 4)));
                        const int orow_i = q0 + quad * 32 + r;
                        if (orow_i < p.Sq)
                            *reinterpret_cast<uint4*>(obase + (int64_t)orow_i * p.o_ss + (c >> 1) * 64 + piece * 8) = val;
                    }
                    __syncwarp();
                }
            }
            // this thread's reads of O are complete before it can arrive on p_full for the next tile's first
            // block, and the next tile's first P V (which overwrites O) waits for that arrival
            ptx::tc_fence_before();
        }
        if (!ok && lane == 0) atomicOr(&g_sdpa_status[0], 64u);
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

template <typename T, int D>
int launch_flash_tc(const SdpaParams& p, cudaStream_t st) {
    using Cfg = FlashCfg<D>;
    constexpr bool is_bf16 = std::is_same<T, __nv_bfloat16>::value;
    CUtensorMap tq, tk, tv;
    if (!make_tmap_bhsd_16bit(&tq, p.q, p.B, p.H, p.Sq, D, p.q_sb, p.q_sh, p.q_ss, FM, is_bf16) ||
        !make_tmap_bhsd_16bit(&tk, p.k, p.B, p.H, p.Skv, D, p.k_sb, p.k_sh, p.k_ss, FN, is_bf16) ||
        !make_tmap_bhsd_16bit(&tv, p.v, p.B, p.H, p.Skv, D, p.v_sb, p.v_sh, p.v_ss, FN, is_bf16))
        return fail(XG_ERR_UNSUPPORTED, "xg_sdpa_fwd: tensor-map encoding failed (strides must be multiples of 8 elements)");
    FlashParams fp;
    fp.mask = p.mask;
    fp.out = p.out;
    fp.o_sb = p.o_sb; fp.o_sh = p.o_sh; fp.o_ss = p.o_ss;
    fp.m_sb = p.m_sb; fp.m_sh = p.m_sh; fp.m_sq = p.m_sq; fp.m_sk = p.m_sk;
    fp.B = (int)p.B; fp.H = (int)p.H; fp.Sq = (int)p.Sq; fp.Skv = (int)p.Skv;  // the caller keeps these below 2^31
    fp.scale = p.scale;
    fp.causal = p.causal;
    const bool masked = p.mask != nullptr || p.Skv % FN != 0 || !(p.scale > 0.f);
    auto kern = masked ? flash_tc_kernel<T, D, true> : flash_tc_kernel<T, D, false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(XG_ERR_LAUNCH, "xg_sdpa_fwd: cannot reserve shared memory: %s", cudaGetErrorString(e));
    }
    const int64_t tiles = p.B * p.H * ((p.Sq + FM - 1) / FM);
    if (tiles > 0x7fffffffLL) return fail(XG_ERR_TOO_LARGE, "xg_sdpa_fwd: too many tiles");
    const int64_t resident = 2LL * num_sms();  // persistent CTAs, two per SM
    const int64_t pairs = (tiles + 1) / 2;      // a CTA takes tiles in neighbouring (heavy, light) pairs
    const unsigned grid = (unsigned)(pairs < resident ? pairs : resident);
    kern<<<grid, kFlashThreads, Cfg::SMEM_BYTES, st>>>(tq, tk, tv, fp);
    return check_launch("xg_sdpa_fwd");
}

// ---------------------------------------------------------------------------------------
// SIMT kernel: one warp per query row, true fp32 arithmetic, any dtype / strides, D <= 256.
// Key rows and value rows are read with coalesced loads (lane l holds elements l + 32 u of the head dim); lane t keeps
// the score of key j0 + t; the output row is spread over the lanes the same way.
// ---------------------------------------------------------------------------------------
constexpr int kSimtWarps = 4;
constexpr int kSimtMaxD = 256;
constexpr int kSimtKeys = 16;  // key / value rows whose loads are in flight together (the loop is latency-bound)

template <typename T>
__global__ void __launch_bounds__(kSimtWarps * 32) sdpa_simt_kernel(const SdpaParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t gr = (int64_t)blockIdx.x * kSimtWarps + warp;  // global query row over (b, h, i)
    if (gr >= p.B * p.H * p.Sq) return;
    const int64_t i = gr % p.Sq;
    const int64_t bh = gr / p.Sq;
    const int64_t h = bh % p.H, b = bh / p.H;
    const int D = (int)p.D;
    const T* qrow = reinterpret_cast<const T*>(p.q) + b * p.q_sb + h * p.q_sh + i * p.q_ss;
    const T* kbase = reinterpret_cast<const T*>(p.k) + b * p.k_sb + h * p.k_sh;
    const T* vbase = reinterpret_cast<const T*>(p.v) + b * p.v_sb + h * p.v_sh;
    const T* mrow = p.mask ? reinterpret_cast<const T*>(p.mask) + b * p.m_sb + h * p.m_sh + i * p.m_sq : nullptr;
    const int nu = (D + 31) / 32;  // head-dim elements (and output columns) per lane
    float qreg[kSimtMaxD / 32];
#pragma unroll
    for (int u = 0; u < kSimtMaxD / 32; ++u) qreg[u] = (lane + 32 * u < D) ? Cvt<T>::to_f(qrow[lane + 32 * u]) : 0.f;
    float o[kSimtMaxD / 32];
#pragma unroll
    for (int u = 0; u < kSimtMaxD / 32; ++u) o[u] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    int64_t kv_end = p.Skv;
    if (p.causal && i + 1 < kv_end) kv_end = i + 1;
    for (int64_t j0 = 0; j0 < kv_end; j0 += 32) {
        const int64_t j = j0 + lane;
        const int cnt = (int)((kv_end - j0) < 32 ? (kv_end - j0) : 32);
        // Scores of keys j0 .. j0+cnt-1. All lanes work on one key at a time, each on its slice of the head dim
        // (coalesced 128-byte loads of the key row, then a warp reduction); sixteen keys are in flight so that
        // the loads and the shuffle chains overlap. Lane t keeps the score of key j0 + t. (A lane walking its own key
        // row would touch 32 different lines per load and saturate the L1 instead.)
        float s = -INFINITY;
        for (int t0 = 0; t0 < cnt; t0 += kSimtKeys) {
            float part[kSimtKeys];
#pragma unroll
            for (int e = 0; e < kSimtKeys; ++e) part[e] = 0.f;
            for (int u = 0; u < nu; ++u) {
                const int d = lane + 32 * u;
                float qv = 0.f;
#pragma unroll
                for (int uu = 0; uu < kSimtMaxD / 32; ++uu)
                    if (uu == u) qv = qreg[uu];
                float kv[kSimtKeys];  // all loads of the group are issued before the first use: one round trip per group
#pragma unroll
                for (int e = 0; e < kSimtKeys; ++e)
                    kv[e] = (t0 + e < cnt && d < D) ? Cvt<T>::to_f(kbase[(j0 + t0 + e) * p.k_ss + d]) : 0.f;
#pragma unroll
                for (int e = 0; e < kSimtKeys; ++e) part[e] = fmaf(qv, kv[e], part[e]);
            }
#pragma unroll
            for (int o2 = 16; o2 > 0; o2 >>= 1)
#pragma unroll
                for (int e = 0; e < kSimtKeys; ++e) part[e] += __shfl_xor_sync(0xffffffffu, part[e], o2);
#pragma unroll
            for (int e = 0; e < kSimtKeys; ++e)
                if (lane == t0 + e) s = part[e] * p.scale;
        }
        if (j < kv_end) {
            if (mrow) s += Cvt<T>::to_f(mrow[j * p.m_sk]);
        } else {
            s = -INFINITY;
        }
        const float m_new = fmaxf(m_run, warp_max(s));
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = expf(m_run - m_use);
        const float pj = expf(s - m_use);
        l_run = l_run * alpha + warp_sum(pj);
#pragma unroll
        for (int u = 0; u < kSimtMaxD / 32; ++u) o[u] *= alpha;
        for (int t0 = 0; t0 < cnt; t0 += kSimtKeys) {  // a group of value rows in flight at a time
            for (int u = 0; u < nu; ++u) {
                const int d = lane + 32 * u;
                float vv[kSimtKeys];
#pragma unroll
                for (int e = 0; e < kSimtKeys; ++e)
                    vv[e] = (t0 + e < cnt && d < D) ? Cvt<T>::to_f(vbase[(j0 + t0 + e) * p.v_ss + d]) : 0.f;
                float a0 = 0.f, a1 = 0.f;
#pragma unroll
                for (int e = 0; e < kSimtKeys; e += 2) {
                    a0 = fmaf(__shfl_sync(0xffffffffu, pj, t0 + e), vv[e], a0);
                    a1 = fmaf(__shfl_sync(0xffffffffu, pj, t0 + e + 1), vv[e + 1], a1);
                }
                // o[u] with a runtime u would leave the registers: select the slot with a compile-time loop
#pragma unroll
                for (int uu = 0; uu < kSimtMaxD / 32; ++uu)
                    if (uu == u) o[uu] += a0 + a1;
            }
        }
        m_run = m_new;
    }
    const float inv_l = 1.0f / l_run;
    T* orow = reinterpret_cast<T*>(p.out) + b * p.o_sb + h * p.o_sh + i * p.o_ss;
#pragma unroll
    for (int u = 0; u < kSimtMaxD / 32; ++u) {
        const int d = lane + 32 * u;
        if (d < D) orow[d] = Cvt<T>::from_f(o[u] * inv_l);
    }
}

// ---------------------------------------------------------------------------------------
// Tiled SIMT kernel: true fp32 arithmetic for head dims 32 / 64 / 128 without an additive mask (the encoder block's
// attention). A CTA owns 16 query rows of one (batch, head): 4 warps x 4 rows. Keys and values pass through shared
// memory in chunks of 128 (each element is read from global memory once per CTA, coalesced, instead of once per query
// row): lane t holds the scores of keys t, t + 32, t + 64, t + 96 for the warp's four rows (64 FMAs per eight 16-byte
// shared-memory loads), the probabilities go back through shared memory, and lane t accumulates output columns t,
// t + 32, ... Online softmax across chunks; a warp reduction per row and chunk.
// ---------------------------------------------------------------------------------------
constexpr int kTileQ = 16;
constexpr int kTileK = 128;
constexpr int kTileThreads = 128;

template <int D>
struct TileCfg {
    static constexpr int KS = D + 4;  // key row stride in floats: an odd multiple of 16 bytes, so that the 16-byte loads of
                                      // eight lanes (eight different keys) fall into 32 different banks
    static constexpr int SMEM_BYTES = (kTileK * KS + kTileK * D + kTileQ * D + kTileQ * kTileK) * 4;
};

template <typename T, int D>
__global__ void __launch_bounds__(kTileThreads) sdpa_tile_kernel(const SdpaParams p) {
    using Cfg = TileCfg<D>;
    constexpr int KS = Cfg::KS;
    constexpr int NU = D / 32;  // output columns per lane
    extern __shared__ __align__(16) float tile_smem[];
    float* Ks = tile_smem;             // [kTileK][KS]
    float* Vs = Ks + kTileK * KS;      // [kTileK][D]
    float* Qs = Vs + kTileK * D;       // [kTileQ][D], pre-multiplied by the scale
    float* Ps = Qs + kTileQ * D;       // [kTileQ][kTileK]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t bh = blockIdx.y;
    const int64_t h = bh % p.H, b = bh / p.H;
    const int q0 = (int)blockIdx.x * kTileQ;
    const int Sq = (int)p.Sq, Skv = (int)p.Skv;
    const T* qbase = reinterpret_cast<const T*>(p.q) + b * p.q_sb + h * p.q_sh;
    const T* kbase = reinterpret_cast<const T*>(p.k) + b * p.k_sb + h * p.k_sh;
    const T* vbase = reinterpret_cast<const T*>(p.v) + b * p.v_sb + h * p.v_sh;

    for (int idx = threadIdx.x; idx < kTileQ * D; idx += kTileThreads) {
        const int r = idx / D, d = idx - r * D;
        Qs[idx] = (q0 + r < Sq) ? Cvt<T>::to_f(qbase[(int64_t)(q0 + r) * p.q_ss + d]) * p.scale : 0.f;
    }
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(kbase) | reinterpret_cast<uintptr_t>(vbase)) & 15u) == 0 &&
                        p.k_ss % (16 / (int)sizeof(T)) == 0 && p.v_ss % (16 / (int)sizeof(T)) == 0;
    int kv_end = Skv;  // keys any row of this CTA can see
    if (p.causal && q0 + kTileQ < kv_end) kv_end = q0 + kTileQ;

    const int row0 = q0 + warp * 4;
    float o[4][NU];
    float m_run[4], l_run[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        m_run[r] = -INFINITY;
        l_run[r] = 0.f;
#pragma unroll
        for (int u = 0; u < NU; ++u) o[r][u] = 0.f;
    }
    const float* qw = Qs + warp * 4 * D;
    float* pw = Ps + warp * 4 * kTileK;

    for (int k0 = 0; k0 < kv_end; k0 += kTileK) {
        __syncthreads();  // the previous chunk has been consumed (first time: Qs is complete)
        // this chunk's keys and values (zeros beyond the last visible key), coalesced along the head dim; 16-byte loads
        // where the rows allow them, many of them in flight per thread (the chunk is a single round trip to L2)
        if (vec_ok) {
            constexpr int EV = 16 / (int)sizeof(T);  // elements per 16-byte load
            constexpr int VPR = D / EV;              // loads per row
#pragma unroll 8
            for (int idx = threadIdx.x; idx < kTileK * VPR; idx += kTileThreads) {
                const int key = idx / VPR, d = (idx - key * VPR) * EV;
                Vec16<T> kv, vv;
                if (k0 + key < kv_end) {
                    kv = ld16(kbase + (int64_t)(k0 + key) * p.k_ss + d);
                    vv = ld16(vbase + (int64_t)(k0 + key) * p.v_ss + d);
                } else {
#pragma unroll
                    for (int e = 0; e < EV; ++e) kv.v[e] = vv.v[e] = Cvt<T>::from_f(0.f);
                }
#pragma unroll
                for (int e = 0; e < EV; e += 4) {
                    *reinterpret_cast<float4*>(Ks + key * KS + d + e) = make_float4(Cvt<T>::to_f(kv.v[e]), Cvt<T>::to_f(kv.v[e + 1]),
                                                                                    Cvt<T>::to_f(kv.v[e + 2]), Cvt<T>::to_f(kv.v[e + 3]));
                    *reinterpret_cast<float4*>(Vs + key * D + d + e) = make_float4(Cvt<T>::to_f(vv.v[e]), Cvt<T>::to_f(vv.v[e + 1]),
                                                                                   Cvt<T>::to_f(vv.v[e + 2]), Cvt<T>::to_f(vv.v[e + 3]));
                }
            }
        } else {
#pragma unroll 4
            for (int idx = threadIdx.x; idx < kTileK * D; idx += kTileThreads) {
                const int key = idx / D, d = idx - key * D;
                const bool in = k0 + key < kv_end;
                Ks[key * KS + d] = in ? Cvt<T>::to_f(kbase[(int64_t)(k0 + key) * p.k_ss + d]) : 0.f;
                Vs[idx] = in ? Cvt<T>::to_f(vbase[(int64_t)(k0 + key) * p.v_ss + d]) : 0.f;
            }
        }
        __syncthreads();
        // scores of keys k0 + lane + 32 i for the warp's four rows
        float sc[4][4];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int i = 0; i < 4; ++i) sc[r][i] = 0.f;
#pragma unroll 4
        for (int d = 0; d < D; d += 4) {
            float4 qv[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) qv[r] = *reinterpret_cast<const float4*>(qw + r * D + d);  // same address in every lane
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 kv = *reinterpret_cast<const float4*>(Ks + (lane + 32 * i) * KS + d);
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    sc[r][i] = fmaf(qv[r].x, kv.x, fmaf(qv[r].y, kv.y, fmaf(qv[r].z, kv.z, fmaf(qv[r].w, kv.w, sc[r][i]))));
            }
        }
        // online softmax per row; the probabilities go to shared memory for the second product
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int row = row0 + r;
            float mx = -INFINITY;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int key = k0 + lane + 32 * i;
                if (key >= Skv || (p.causal && key > row)) sc[r][i] = -INFINITY;
                mx = fmaxf(mx, sc[r][i]);
            }
            const float m_new = fmaxf(m_run[r], warp_max(mx));
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = expf(m_run[r] - m_use);
            float part = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float pj = expf(sc[r][i] - m_use);
                part += pj;
                pw[r * kTileK + lane + 32 * i] = pj;
            }
            l_run[r] = l_run[r] * alpha + warp_sum(part);
            m_run[r] = m_new;
#pragma unroll
            for (int u = 0; u < NU; ++u) o[r][u] *= alpha;
        }
        __syncwarp();
        // o += P V: four keys per step (the probabilities of a row as one 16-byte load, the same in every lane)
        int cnt = kv_end - k0;
        if (cnt > kTileK) cnt = kTileK;
        for (int k = 0; k < cnt; k += 4) {
            float4 pv[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) pv[r] = *reinterpret_cast<const float4*>(pw + r * kTileK + k);
#pragma unroll
            for (int u = 0; u < NU; ++u) {
                const float v0 = Vs[(k + 0) * D + lane + 32 * u], v1 = Vs[(k + 1) * D + lane + 32 * u];
                const float v2 = Vs[(k + 2) * D + lane + 32 * u], v3 = Vs[(k + 3) * D + lane + 32 * u];
#pragma unroll
                for (int r = 0; r < 4; ++r)
                    o[r][u] = fmaf(pv[r].x, v0, fmaf(pv[r].y, v1, fmaf(pv[r].z, v2, fmaf(pv[r].w, v3, o[r][u]))));
            }
        }
    }
    T* obase = reinterpret_cast<T*>(p.out) + b * p.o_sb + h * p.o_sh;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        if (row0 + r >= Sq) continue;
        const float inv_l = 1.0f / l_run[r];
#pragma unroll
        for (int u = 0; u < NU; ++u) obase[(int64_t)(row0 + r) * p.o_ss + lane + 32 * u] = Cvt<T>::from_f(o[r][u] * inv_l);
    }
}

template <typename T, int D>
int launch_tile(const SdpaParams& p, cudaStream_t st) {
    using Cfg = TileCfg<D>;
    auto kern = sdpa_tile_kernel<T, D>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(XG_ERR_LAUNCH, "xg_sdpa_fwd: cannot reserve shared memory: %s", cudaGetErrorString(e));
    }
    const int64_t qt = (p.Sq + kTileQ - 1) / kTileQ, bh = p.B * p.H;
    if (qt > 0x7fffffffLL || bh > 65535) return -1;  // the caller falls back to the row-per-warp kernel
    kern<<<dim3((unsigned)qt, (unsigned)bh), kTileThreads, Cfg::SMEM_BYTES, st>>>(p);
    return check_launch("xg_sdpa_fwd");
}

template <typename T>
int launch_tile_any(const SdpaParams& p, cudaStream_t st) {
    switch ((int)p.D) {
        case 32: return launch_tile<T, 32>(p, st);
        case 64: return launch_tile<T, 64>(p, st);
        case 128: return launch_tile<T, 128>(p, st);
        default: return -1;
    }
}

template <typename T>
int launch_simt(const SdpaParams& p, cudaStream_t st) {
    const int64_t rows = p.B * p.H * p.Sq;
    const int64_t grid = (rows + kSimtWarps - 1) / kSimtWarps;
    if (grid > 0x7fffffffLL) return fail(XG_ERR_TOO_LARGE, "xg_sdpa_fwd: too many rows");
    sdpa_simt_kernel<T><<<(unsigned)grid, kSimtWarps * 32, 0, st>>>(p);
    return check_launch("xg_sdpa_fwd");
}

}  // namespace
}  // namespace xg

namespace xg {
int read_sdpa_status(unsigned int* host_out, int reset) {
    unsigned int v[4] = {0, 0, 0, 0};
    if (cudaMemcpyFromSymbol(v, g_sdpa_status, sizeof(v)) != cudaSuccess) {
        cudaGetLastError();
        return fail(XG_ERR_DEVICE, "xg_tc_status: cannot read device status");
    }
    *host_out = v[0];
    if (reset && v[0] != 0) {
        unsigned int z[4] = {0, 0, 0, 0};
        cudaMemcpyToSymbol(g_sdpa_status, z, sizeof(z));
    }
    return XG_OK;
}
}  // namespace xg

extern "C" int xg_sdpa_fwd(const void* q, const void* k, const void* v, const void* mask, void* out, int64_t B, int64_t H,
                           int64_t Sq, int64_t Skv, int64_t D, const int64_t* q_strides3, const int64_t* k_strides3,
                           const int64_t* v_strides3, const int64_t* o_strides3, const int64_t* mask_strides4, float scale,
                           int causal, int dtype, void* stream) {
    using namespace xg;
    if (!q || !k || !v || !out || !q_strides3 || !k_strides3 || !v_strides3 || !o_strides3)
        return fail(XG_ERR_INVALID_ARG, "xg_sdpa_fwd: null pointer");
    if (mask && !mask_strides4) return fail(XG_ERR_INVALID_ARG, "xg_sdpa_fwd: mask given without strides");
    if (B < 0 || H < 0 || Sq < 0 || Skv < 0 || D <= 0) return fail(XG_ERR_INVALID_ARG, "xg_sdpa_fwd: bad extents");
    if (dtype_size(dtype) == 0) return fail(XG_ERR_INVALID_ARG, "xg_sdpa_fwd: bad dtype %d", dtype);
    if (D > kSimtMaxD) return fail(XG_ERR_UNSUPPORTED, "xg_sdpa_fwd: head_dim %lld > %d", (long long)D, kSimtMaxD);
    if (B * H * Sq == 0) return XG_OK;
    SdpaParams p;
    p.q = q; p.k = k; p.v = v; p.mask = mask; p.out = out;
    p.B = B; p.H = H; p.Sq = Sq; p.Skv = Skv; p.D = D;
    p.q_sb = q_strides3[0]; p.q_sh = q_strides3[1]; p.q_ss = q_strides3[2];
    p.k_sb = k_strides3[0]; p.k_sh = k_strides3[1]; p.k_ss = k_strides3[2];
    p.v_sb = v_strides3[0]; p.v_sh = v_strides3[1]; p.v_ss = v_strides3[2];
    p.o_sb = o_strides3[0]; p.o_sh = o_strides3[1]; p.o_ss = o_strides3[2];
    p.m_sb = mask ? mask_strides4[0] : 0; p.m_sh = mask ? mask_strides4[1] : 0;
    p.m_sq = mask ? mask_strides4[2] : 0; p.m_sk = mask ? mask_strides4[3] : 0;
    p.scale = scale;
    p.causal = causal ? 1 : 0;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

    auto tma_ok = [&](const void* ptr, int64_t sb, int64_t sh, int64_t ss, int64_t S) {
        auto okst = [&](int64_t s, int64_t extent) { return extent == 1 || (s > 0 && s % 8 == 0); };
        return aligned16(ptr) && okst(ss, S) && okst(sh, H) && okst(sb, B);
    };
    const bool tc = (dtype != XG_F32) && (D == 64 || D == 128) && Skv > 0 && tma_ok(q, p.q_sb, p.q_sh, p.q_ss, Sq) &&
                    tma_ok(k, p.k_sb, p.k_sh, p.k_ss, Skv) && tma_ok(v, p.v_sb, p.v_sh, p.v_ss, Skv) && aligned16(out) &&
                    p.o_ss % 8 == 0 && p.o_sh % 8 == 0 && p.o_sb % 8 == 0 && Sq < 0x7fffff00LL && Skv < 0x7fffff00LL;
    if (tc) {
        if (dtype == XG_BF16) return D == 128 ? launch_flash_tc<__nv_bfloat16, 128>(p, st) : launch_flash_tc<__nv_bfloat16, 64>(p, st);
        return D == 128 ? launch_flash_tc<__half, 128>(p, st) : launch_flash_tc<__half, 64>(p, st);
    }
    if (mask == nullptr && Sq < 0x7fffff00LL && Skv < 0x7fffff00LL) {  // -1: not a shape the tiled kernel takes
        int rc = -1;
        switch (dtype) {
            case XG_F32: rc = launch_tile_any<float>(p, st); break;
            case XG_BF16: rc = launch_tile_any<__nv_bfloat16>(p, st); break;
            default: rc = launch_tile_any<__half>(p, st); break;
        }
        if (rc != -1) return rc;
    }
    switch (dtype) {
        case XG_F32: return launch_simt<float>(p, st);
        case XG_BF16: return launch_simt<__nv_bfloat16>(p, st);
        default: return launch_simt<__half>(p, st);
    }
}
