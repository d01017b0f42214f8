// Attention over the paged cache on the 5th-generation tensor cores: a prefill kernel (portions of
// many tokens) and a decode kernel (few tokens per request, keys split into ranges and planned once
// per step).  Common to both: key/value pages arrive by TMA (cp.async.bulk.tensor, 128-byte swizzle,
// one box per page and 64-column half) in rings of shared-memory stages guarded by mbarriers; every
// tcgen05.mma is issued by one thread of an issuer warp and frees its stages with tcgen05.commit; the
// roles meet only through mbarriers; S = Q K^T, P and O live in tensor memory; the softmax of a row
// runs in registers (float32, base 2), and the running maximum is only moved when it grows by more
// than 2^8, so O is rescaled (tcgen05.ld / tcgen05.st) rarely; the final O / l is exact either way.
// Value rows outside the request's visible keys are zeroed in shared memory before they are
// multiplied, so stale or poisoned pages cannot reach a result.  Every mbarrier wait is bounded
// (XB_ERR_WAIT in the error word on expiry, then the CTA frees its TMEM and leaves).
// Head sizes: multiples of 16 up to 128.  Page sizes: powers of two from 8.
#include "attention_common.cuh"
#include "tc_common.cuh"

namespace {

using namespace xbtc;

constexpr int QT = 128;  // queries per CTA
constexpr int KT = 64;   // keys per tile
constexpr float RESCALE_STEP = 8.f;  // the row maximum moves only when it grows by more than 2^8

// ------------------------------------------------------------------------------------------------
// prefill: 128 queries of two query heads per work item; a CTA per SM works through a list of items
// ------------------------------------------------------------------------------------------------
// A work item is 128 queries of one request's portion for TWO query heads that share their key/value
// head, so a key/value tile is loaded once for both (a tile per 8 MFLOP instead of 4) and the rings are
// three stages deep (a tile's way from memory is longer than two; a fourth stage gave its room to
// the output staging).  The host shares the step's items out
// among at most one CTA per SM, longest first onto the least loaded CTA (xb_attn_prefill_work), so that
// SMs finish together whatever the lengths are, and a CTA that stays on its SM overlaps the end of an
// item with the start of the next: the key pages of the next item are requested as soon as ring stages
// are free, its Q as soon as the last Q K^T of this item has read the old one, and its first scores are
// computed while this item's output leaves.
//   warps 0..3: softmax of head A (one row per thread), warps 4..7: softmax of head B,
//   warp 8: TMA producer of the key pages, warp 10: of the value pages (one lane per page box; the page
//   ids of the next tile are fetched while this one is issued),
//   warp 9: loads Q (both heads) and issues S_A, S_B = Q K^T of every tile; warp 11: issues O_A += P_A V
//   and O_B += P_B V (two issuers, so that the waits of one do not hold up the products of the other; P
//   lies in tensor memory over the scores it came from, so the first waits for the second before it
//   reuses a score buffer).
// Shared memory (1024-byte aligned): Q [2 heads][DP/64][128 rows][64], then three stages of K and V
// [DP/64][64 keys][64]; every [rows][64] piece is a tile of 128-byte rows whose 16-byte chunks are
// XOR-ed with row & 7; then the barriers; then 4 KB per softmax warp and 64-column half through which
// full output tiles leave by TMA stores (a warp's 32 rows; nobody waits for the stores until the warp
// needs the space for its next item).
// Tensor memory (all 512 columns): S_A[0], S_A[1], S_B[0], S_B[1] at 0, 64, 128, 192; O_A at 256, O_B at 384.
// Barriers carry on from item to item: their parities come from running counts of tiles (of all tiles
// for the rings, of a head's tiles for what belongs to a head) and of items.
// With an odd number of query heads per key/value head the last item of the group has one head and the
// second softmax warpgroup sits it out; the host also makes items of one head when two-head items would be
// too few to fill the SMs (short portions, few heads).
constexpr int PREFILL_STAGES = 3;
constexpr int PREFILL_THREADS = 384;
constexpr int PREFILL_ITEM_INTS = 4;   // portion, query tile, first query head, heads (2 of one key/value head, or 1)

// What the roles of a CTA derive, each for itself, from an item of the work list.
struct PrefillItem {
    int g, h0, nhd;               // key/value head, first query head, heads (2, or 1)
    int rows, t0, p0;             // queries, their first row in q / out, the first one's position
    int first_key, last_key, kt_first, iters;
    const int* table;
};

__device__ __forceinline__ PrefillItem prefill_item(const int* __restrict__ item, const int* __restrict__ q_start,
                                                    const int* __restrict__ start_pos, const int* __restrict__ block_table,
                                                    int table_stride, int nh, int nkv, int window) {
    PrefillItem w;
    const int b = item[0], tile = item[1];
    w.h0 = item[2];
    // one of two values, and written so: the loops over an item's heads are then compiled without a case of
    // no head at all, which costs the issuing threads 9 % of a long item's time
    w.nhd = item[3] == 2 ? 2 : 1;
    w.g = w.h0 / (nh / nkv);
    const int n = q_start[b + 1] - q_start[b];
    const int row0 = tile * QT;
    w.rows = min(QT, n - row0);
    w.t0 = q_start[b] + row0;
    w.p0 = start_pos[b] + row0;
    w.last_key = w.p0 + w.rows - 1;
    w.first_key = window > 0 ? max(0, w.p0 - window + 1) : 0;
    w.table = block_table + (size_t)b * table_stride;
    w.kt_first = w.first_key / KT;
    w.iters = w.last_key / KT - w.kt_first + 1;
    return w;
}

// `work`: [ctas + 1] offsets into the items that follow them, PREFILL_ITEM_INTS int32 each; CTA c takes
// items work[c] .. work[c + 1] - 1 in that order.
template <int DP>
__global__ void __launch_bounds__(PREFILL_THREADS)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                       __nv_bfloat16* __restrict__ out, const int* __restrict__ q_start, const int* __restrict__ start_pos,
                       const int* __restrict__ block_table, int table_stride, int nh, int nkv, int d,
                       int ps, int ps_shift, int num_pages, int window, float scale_log2,
                       const int* __restrict__ work, int* err) {
    constexpr int HALVES = DP / 64, NS = PREFILL_STAGES;
    constexpr uint32_t Q_ONE = HALVES * QT * 128, Q_BYTES = 2 * Q_ONE;
    constexpr uint32_t KV_HALF = KT * 128, KV_BYTES = HALVES * KV_HALF, STAGE_BYTES = 2 * KV_BYTES;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t q_sm = base, kv_sm = base + Q_BYTES;
    // barriers, 8 bytes each: k_full[4] k_empty[4] v_full[4] v_empty[4] (NS of each in use) s_ready[head][2]
    // pv_done[head][2] p_ready[head] q_full bar_o q_empty; then four words; the output staging 1024 bytes after BAR_OFF
    constexpr uint32_t BAR_OFF = Q_BYTES + NS * STAGE_BYTES, OUT_OFF = BAR_OFF + 1024;
    const uint32_t bars = base + BAR_OFF;
    const uint32_t k_full0 = bars, k_empty0 = bars + 32, v_full0 = bars + 64, v_empty0 = bars + 96;
    const uint32_t s_ready0 = bars + 128, pv_done0 = bars + 160, p_ready0 = bars + 192;
    const uint32_t q_full = bars + 208, bar_o = bars + 216, q_empty = bars + 224;
    volatile uint32_t* words = reinterpret_cast<volatile uint32_t*>(smem_raw + BAR_OFF + 240);  // tmem, -, -, dead
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();

    // what follows until the wait reads only what the host sent before the step's first kernel
    const int ctas = (int)gridDim.x;
    int item_begin = work[blockIdx.x], item_end = work[blockIdx.x + 1];
    const int* const items = work + ctas + 1;
    if (threadIdx.x == 0) {
        if (base & 1023u) atomicOr(err, XB_ERR_WAIT);  // the swizzle needs a 1024-byte aligned window
        words[3] = 0;
        for (int i = 0; i < 4 * 4; ++i) mbar_init(bars + 8 * i, 1);         // k_full, k_empty, v_full, v_empty
        for (int i = 0; i < 4; ++i) mbar_init(s_ready0 + 8 * i, 1);
        for (int i = 0; i < 2; ++i) mbar_init(p_ready0 + 8 * i, 128);
        for (int i = 0; i < 4; ++i) mbar_init(pv_done0 + 8 * i, 1);
        mbar_init(q_full, 1);
        mbar_init(bar_o, 1);
        mbar_init(q_empty, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // an earlier CTA gave up: do not pile on
    if (*reinterpret_cast<volatile int*>(err) & XB_ERR_WAIT) item_end = item_begin;
    __syncthreads();
    if (item_end <= item_begin || (base & 1023u)) {
        pdl_wait();   // a kernel that depends on this one may rely on every block having waited
        return;
    }
    constexpr uint32_t TMEM_COLS = 512;
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(const_cast<uint32_t*>(&words[0]))), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = words[0];
    pdl_wait();   // q and the new keys and values come from the kernel before

    const int box_rows = ps < KT ? ps : KT;
    auto item_at = [&](int k) {
        return prefill_item(items + (size_t)k * PREFILL_ITEM_INTS, q_start, start_pos, block_table, table_stride, nh, nkv, window);
    };
    if (warp == 8 || warp == 10) {
        // ---- producers of key pages (warp 8) and value pages (warp 10), item after item ----------------------
        const bool is_v = warp == 10;
        const uint32_t full0 = is_v ? v_full0 : k_full0, empty0 = is_v ? v_empty0 : k_empty0;
        const CUtensorMap* map = is_v ? &map_v : &map_k;
        int s = 0;            // the ring stage of the next tile, over all items
        uint32_t ph = 0;      // parity of the number of times the ring has been gone round
        bool rounds = false;  // it has been gone round at least once
        bool ok = true;
        for (int k = item_begin; k < item_end && ok; ++k) {
            const PrefillItem w = item_at(k);
            const int boxes = (KT / box_rows) * HALVES;     // at most 16: one lane each
            const int bi = lane / HALVES, hf = lane % HALVES;
            auto page_of = [&](int it) -> int {             // the page of this lane's box in tile `it`, -1: nothing to load
                const int j = (w.kt_first + it) * KT + bi * box_rows;
                if (it >= w.iters || lane >= boxes || j > w.last_key || j + box_rows - 1 < w.first_key) return -1;
                const int page = w.table[j >> ps_shift];
                if (page < 0 || page >= num_pages) {
                    atomicOr(err, XB_ERR_BAD_PAGE);
                    return -1;
                }
                return page;
            };
            int page_next = page_of(0);
            for (int it = 0; it < w.iters; ++it) {
                const int page = page_next;
                // s = (tiles so far) % NS and the parity of their quotient run along: no division per tile
                if (rounds && !__all_sync(0xffffffffu, mbar_wait(empty0 + 8 * s, ph ^ 1u, err))) {
                    words[3] = 1;
                    ok = false;
                    break;
                }
                const uint32_t nb = __popc(__ballot_sync(0xffffffffu, page >= 0));
                if (lane == 0) mbar_expect_tx(full0 + 8 * s, nb * box_rows * 128);
                __syncwarp();
                if (page >= 0) {
                    const int j = (w.kt_first + it) * KT + bi * box_rows;
                    const uint32_t dst = kv_sm + s * STAGE_BYTES + (is_v ? KV_BYTES : 0u) + hf * KV_HALF + bi * box_rows * 128;
                    tma_load_2d(dst, map, hf * 64, (page * nkv + w.g) * ps + (j & (ps - 1)), full0 + 8 * s);
                }
                page_next = page_of(it + 1);
                if (++s == NS) {
                    s = 0;
                    ph ^= 1u;
                    rounds = true;
                }
            }
        }
    } else if (warp == 9) {
        // ---- Q loads and S = Q K^T, both heads, tile after tile, item after item: the whole warp walks the loop
        // (its values stay uniform), one lane issues -----------------------------------------------------------
        {
            const bool leader = lane == 0;
            const uint32_t idesc_s = umma_idesc(KT, 0);
            const uint64_t dq0 = umma_desc(q_sm, 16, 1024), dk0 = umma_desc(kv_sm, 16, 1024);
            auto load_q = [&](const PrefillItem& w) {
                if (leader) {
                    mbar_expect_tx(q_full, (uint32_t)w.nhd * Q_ONE);
                    for (int hd = 0; hd < w.nhd; ++hd)
#pragma unroll
                        for (int hf = 0; hf < HALVES; ++hf)
                            tma_load_3d(q_sm + hd * Q_ONE + hf * QT * 128, &map_q, hf * 64, w.h0 + hd, w.t0, q_full);
                }
                __syncwarp();
            };
            int s = 0, Th[2] = {0, 0};   // ring stage of the next tile (over all items), tiles of each head so far
            uint32_t ph = 0;               // parity of the times the ring has been gone round
            bool ok = true;
            PrefillItem w = item_at(item_begin);
            load_q(w);
            for (int k = item_begin; k < item_end && ok; ++k) {
                const int I = k - item_begin;
                ok = __all_sync(0xffffffffu, mbar_wait(q_full, (uint32_t)I & 1u, err, true));
                for (int it = 0; it < w.iters && ok; ++it) {
                    ok = __all_sync(0xffffffffu, mbar_wait(k_full0 + 8 * s, ph, err, true));
                    const uint64_t dk = dk0 + (uint64_t)((s * STAGE_BYTES) >> 4);
#pragma unroll
                    for (int hd = 0; hd < 2; ++hd) {
                        if (hd >= w.nhd) break;
                        const int th = Th[hd] + it, sb = th & 1;
                        // S[sb] of this head held the scores and then P of its tile th - 2: that P V must have read it
                        ok = ok && (th < 2 || __all_sync(0xffffffffu, mbar_wait(pv_done0 + 8 * (2 * hd + sb), ((th >> 1) - 1) & 1, err, true)));
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint64_t dq = dq0 + (uint64_t)((hd * Q_ONE) >> 4);
                        if (leader) {
#pragma unroll
                            for (int kk = 0; kk < DP / 16; ++kk) {
                                const uint32_t off = (kk >> 2), inner = (kk & 3) * 32;
                                umma_bf16(tmem + (uint32_t)(hd * 128 + sb * 64), dq + (uint64_t)((off * QT * 128 + inner) >> 4),
                                          dk + (uint64_t)((off * KV_HALF + inner) >> 4), idesc_s, kk ? 1u : 0u);
                            }
                            umma_commit(s_ready0 + 8 * (2 * hd + sb));
                        }
                        __syncwarp();
                    }
                    if (!ok) break;
                    if (leader) umma_commit(k_empty0 + 8 * s);   // the key stage is free once both products have completed
                    __syncwarp();
                    if (++s == NS) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
                if (!ok) break;
                Th[0] += w.iters;
                if (w.nhd == 2) Th[1] += w.iters;
                if (k + 1 < item_end) {
                    // the next item's Q goes where this one's lies: once every product that reads it has completed
                    if (leader) umma_commit(q_empty);
                    __syncwarp();
                    ok = __all_sync(0xffffffffu, mbar_wait(q_empty, (uint32_t)I & 1u, err, true));
                    if (ok) {
                        w = item_at(k + 1);
                        load_q(w);
                    }
                }
            }
            if (!ok) words[3] = 1;
        }
    } else if (warp == 11) {
        // ---- issuer of O += P V, both heads, tile after tile, item after item (the whole warp walks, one lane issues)
        {
            const bool leader = lane == 0;
            const uint32_t idesc_o = umma_idesc(DP, 1);
            const uint64_t dv0 = umma_desc(kv_sm + KV_BYTES, KV_HALF, 1024);
            int s = 0, Th[2] = {0, 0};   // ring stage of the next tile (over all items), tiles of each head so far
            uint32_t ph = 0;               // parity of the times the ring has been gone round
            bool ok = true;
            for (int k = item_begin; k < item_end && ok; ++k) {
                const PrefillItem w = item_at(k);
                for (int it = 0; it < w.iters && ok; ++it) {
                    ok = __all_sync(0xffffffffu, mbar_wait(v_full0 + 8 * s, ph, err, true));
                    const uint64_t dv = dv0 + (uint64_t)((s * STAGE_BYTES) >> 4);
#pragma unroll
                    for (int hd = 0; hd < 2; ++hd) {
                        if (hd >= w.nhd) break;
                        const int th = Th[hd] + it, sb = th & 1;
                        ok = ok && __all_sync(0xffffffffu, mbar_wait(p_ready0 + 8 * hd, th & 1, err, true));   // P written, V rows zeroed, O rescaled
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        // A = P [128 x 64 keys] in tensor memory (over the scores it came from), B = V [64 keys x DP]
                        // MN-major (halves 64 columns apart); the item's first tile overwrites O
                        const uint32_t tp = tmem + (uint32_t)(hd * 128 + sb * 64);
                        if (leader) {
#pragma unroll
                            for (int kk = 0; kk < KT / 16; ++kk)
                                umma_bf16_ta(tmem + (uint32_t)(256 + hd * 128), tp + (uint32_t)(kk * 8), dv + (uint64_t)((kk * 2048) >> 4),
                                             idesc_o, (it | kk) ? 1u : 0u);
                            umma_commit(pv_done0 + 8 * (2 * hd + sb));   // P, its score buffer and O of this head are free again
                        }
                        __syncwarp();
                    }
                    if (!ok) break;
                    if (leader) {
                        umma_commit(v_empty0 + 8 * s);           // and so is the value stage
                        if (it + 1 == w.iters) umma_commit(bar_o);
                    }
                    __syncwarp();
                    if (++s == NS) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
                Th[0] += w.iters;
                if (w.nhd == 2) Th[1] += w.iters;
            }
            if (!ok) words[3] = 1;
        }
    } else if (warp < 8) {
        // ---- softmax: one query row per thread, warps 0..3 for the first head, 4..7 for the second -------------
        const int hd = warp >> 2, r = (int)threadIdx.x & 127;
        const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tmem_s = tmem + (uint32_t)(hd * 128), tmem_o = tmem + (uint32_t)(256 + hd * 128);
        const uint32_t my_s_ready = s_ready0 + 16 * hd;
        const uint32_t my_p_ready = p_ready0 + 8 * hd, my_pv_done = pv_done0 + 16 * hd;
        // this warp's output staging: 32 rows of each 64-column half, swizzled as a TMA box wants them
        unsigned char* const stage = smem_raw + OUT_OFF + warp * (HALVES * 4096);
        const uint32_t stage_sm = base + OUT_OFF + warp * (HALVES * 4096);
        int T = 0, Th = 0;   // tiles of the items before this one: all of them, and those this head took part in
        bool alive = true;
        for (int k = item_begin; k < item_end && alive; ++k) {
            const PrefillItem w = item_at(k);
            const int I = k - item_begin;
            if (hd >= w.nhd) {   // an item of one head: the second warpgroup sits it out
                T += w.iters;
                continue;
            }
            const int iters = w.iters, kt_first = w.kt_first, first_key = w.first_key, last_key = w.last_key, p0 = w.p0;
            const int rows = w.rows, t0 = w.t0, h0 = w.h0;
            const int my_pos = p0 + r;
            float m_ref = -INFINITY, l = 0.f;
            for (int it = 0; it < iters; ++it) {
                const int th = Th + it, sb = th & 1, gt = T + it, st = gt % NS, key0 = (kt_first + it) * KT;
                // every wait's verdict is made warp-wide: tcgen05.ld / .st below need the whole warp
                if (!__all_sync(0xffffffffu, mbar_wait(my_s_ready + 8 * sb, (th >> 1) & 1, err))) {
                    alive = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                float sc[64];
                {
                    uint32_t ra[32], rb[32];
                    tmem_ld32_nowait(tmem_s + sb * 64 + lane_addr, ra);
                    tmem_ld32_nowait(tmem_s + sb * 64 + lane_addr + 32, rb);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    #pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        sc[i] = __uint_as_float(ra[i]);
                        sc[32 + i] = __uint_as_float(rb[i]);
                    }
                }
                const bool edge = key0 + KT - 1 > p0 || key0 + KT - 1 > last_key || key0 < first_key ||
                                  (window > 0 && key0 < p0 + QT - 1 - window + 1);
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                if (edge) {
    #pragma unroll
                    for (int i = 0; i < 64; ++i) {
                        const int j = key0 + i;
                        const bool ok = j <= my_pos && j <= last_key && (window <= 0 || j > my_pos - window);
                        sc[i] = ok ? sc[i] : -INFINITY;
                    }
                }
    #pragma unroll
                for (int i = 0; i < 64; i += 8) {
                    mx4[0] = max3(mx4[0], sc[i], sc[i + 1]);
                    mx4[1] = max3(mx4[1], sc[i + 2], sc[i + 3]);
                    mx4[2] = max3(mx4[2], sc[i + 4], sc[i + 5]);
                    mx4[3] = max3(mx4[3], sc[i + 6], sc[i + 7]);
                }
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
                // move the reference maximum only when the row's maximum outgrows it by more than 2^8
                float corr = 1.f;
                int moved = 0;
                if (mx > m_ref + RESCALE_STEP) {
                    corr = m_ref == -INFINITY ? 0.f : ex2(m_ref - mx);
                    m_ref = mx;
                    moved = it > 0;
                }
                const float m_neg = m_ref == -INFINITY ? 0.f : -m_ref;
                const f32x2 scale2 = pack2(scale_log2, scale_log2), mneg2 = pack2(m_neg, m_neg);
                f32x2 sum_a = pack2(0.f, 0.f), sum_b = pack2(0.f, 0.f);
                uint32_t pk[32];   // the row of P: two bfloat16 per word, in the order of the keys
    #pragma unroll
                for (int c8 = 0; c8 < 8; ++c8) {
                    float x[8], e[8];
    #pragma unroll
                    for (int i = 0; i < 8; i += 2)
                        unpack2(fma2(pack2(sc[c8 * 8 + i], sc[c8 * 8 + i + 1]), scale2, mneg2), x[i], x[i + 1]);
    #pragma unroll
                    for (int i = 0; i < 8; ++i)
                        if ((i & 3) != 3) e[i] = ex2(x[i]);
                    ex2_poly2(x[3], x[7], e[3], e[7]);
                    sum_a = add2(sum_a, add2(pack2(e[0], e[1]), pack2(e[2], e[3])));
                    sum_b = add2(sum_b, add2(pack2(e[4], e[5]), pack2(e[6], e[7])));
                    pk[c8 * 4] = pack_bf16(e[0], e[1]);
                    pk[c8 * 4 + 1] = pack_bf16(e[2], e[3]);
                    pk[c8 * 4 + 2] = pack_bf16(e[4], e[5]);
                    pk[c8 * 4 + 3] = pack_bf16(e[6], e[7]);
                }
                float s0, s1, s2, s3;
                unpack2(sum_a, s0, s1);
                unpack2(sum_b, s2, s3);
                l = l * corr + ((s0 + s1) + (s2 + s3));
                // P goes where the scores were: they are in registers, and the P V that read these columns two tiles
                // ago ran before the Q K^T that wrote them
                tmem_st32_u(tmem_s + sb * 64 + lane_addr, pk);
                // value rows outside the visible keys become zeros (only tiles at the ends of the range): the first
                // head's threads do it; the second head's P V is issued after the first's, so it sees them too
                if (hd == 0 && (key0 < first_key || key0 + KT - 1 > last_key)) {
                    if (r < KT) {
                        mbar_wait(v_full0 + 8 * st, (gt / NS) & 1, err);   // orders these writes after the TMA's
                        const int j = key0 + r;
                        if (j < first_key || j > last_key) {
    #pragma unroll
                            for (int hf = 0; hf < HALVES; ++hf) {
                                uint4* vr = reinterpret_cast<uint4*>(smem_raw + Q_BYTES + st * STAGE_BYTES + KV_BYTES + hf * KV_HALF + r * 128);
    #pragma unroll
                                for (int c8 = 0; c8 < 8; ++c8) vr[c8] = make_uint4(0, 0, 0, 0);
                            }
                        }
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the zeroed rows: visible to the MMA
                    }
                }
                // rescale O where a row's reference maximum moved (rare after the first tiles); tcgen05.ld / .st
                // are warp-wide: a warp rescales when any of its rows moved, the other rows by 1.
                // The previous tile's P V of this head has to be complete before O is touched, and before this tile
                // is announced at all: the issuer waits for the announcements by their parity, so a head must never
                // be two of them ahead of it.
                if (it > 0 && !__all_sync(0xffffffffu, mbar_wait(my_pv_done + 8 * (sb ^ 1), ((th - 1) >> 1) & 1, err))) {
                    alive = false;
                    break;
                }
                if (__any_sync(0xffffffffu, moved)) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const float f = moved ? corr : 1.f;
    #pragma unroll
                    for (int c0 = 0; c0 < DP; c0 += 32) {
                        float o[32];
                        tmem_ld32(tmem_o + lane_addr + c0, o);
    #pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] *= f;
                        tmem_st32(tmem_o + lane_addr + c0, o);
                    }
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");   // P (and O) are in tensor memory
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(my_p_ready);
            }
            // ---- O / l -> out -----------------------------------------------------------------------------------
            if (alive) alive = mbar_wait(bar_o, (uint32_t)I & 1u, err);
            alive = __all_sync(0xffffffffu, alive);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (alive && rows == QT) {
                // a full tile: a warp writes its 32 rows of a 64-column half, swizzled, into its staging space and
                // one thread stores them with a TMA copy: whole lines reach the memory instead of 16 bytes per row
                // and instruction.  Meanwhile the issuers are at work on the next item.
                const float inv = l > 0.f ? 1.f / l : 0.f;
                const int rr = lane;   // row within the warp's 32
                if (lane == 0) tma_store_wait_read();   // the stores of this warp's item before have read the staging space
                __syncwarp();
#pragma unroll
                for (int c0 = 0; c0 < DP; c0 += 32) {
                    float o[32];
                    tmem_ld32(tmem_o + lane_addr + c0, o);
#pragma unroll
                    for (int c8 = 0; c8 < 4; ++c8) {
                        const int cc = (c0 & 63) / 8 + c8;   // 16-byte chunk of the half's row
                        uint4 v;
                        v.x = pack_bf16(o[c8 * 8] * inv, o[c8 * 8 + 1] * inv);
                        v.y = pack_bf16(o[c8 * 8 + 2] * inv, o[c8 * 8 + 3] * inv);
                        v.z = pack_bf16(o[c8 * 8 + 4] * inv, o[c8 * 8 + 5] * inv);
                        v.w = pack_bf16(o[c8 * 8 + 6] * inv, o[c8 * 8 + 7] * inv);
                        *reinterpret_cast<uint4*>(stage + (c0 >> 6) * 4096 + rr * 128 + ((cc ^ (rr & 7)) << 4)) = v;
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
#pragma unroll
                    for (int hf = 0; hf < HALVES; ++hf)
                        if (hf * 64 < d) tma_store_3d(&map_o, stage_sm + hf * 4096, hf * 64, h0 + hd, t0 + (warp & 3) * 32);
                    tma_store_commit();
                }
            } else if (alive) {
                const float inv = l > 0.f ? 1.f / l : 0.f;
                const bool valid = r < rows;
                __nv_bfloat16* dst = out + ((size_t)(t0 + r) * nh + h0 + hd) * d;
#pragma unroll
                for (int c0 = 0; c0 < DP; c0 += 32) {
                    float o[32];
                    tmem_ld32(tmem_o + lane_addr + c0, o);   // warp-wide, whatever `valid` is
                    if (valid) {
#pragma unroll
                        for (int c8 = 0; c8 < 4; ++c8) {
                            const int c = c0 + c8 * 8;
                            if (c < d) {
                                uint4 pk;
                                pk.x = pack_bf16(o[c8 * 8] * inv, o[c8 * 8 + 1] * inv);
                                pk.y = pack_bf16(o[c8 * 8 + 2] * inv, o[c8 * 8 + 3] * inv);
                                pk.z = pack_bf16(o[c8 * 8 + 4] * inv, o[c8 * 8 + 5] * inv);
                                pk.w = pack_bf16(o[c8 * 8 + 6] * inv, o[c8 * 8 + 7] * inv);
                                *reinterpret_cast<uint4*>(dst + c) = pk;
                            }
                        }
                    }
                }
            }
            // the reads of O above come before this head's next announcement (and so before the product that
            // overwrites O): the fence stands in front of that arrive, in the tile loop
            T += iters;
            Th += iters;
        }
        if (lane == 0) tma_store_wait_all();   // the last stores have left before the block does
        if (!alive) words[3] = 1;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// decode: few tokens per request, keys split into ranges
// ------------------------------------------------------------------------------------------------
constexpr int DEC_ROWS = 16;    // query heads of one key/value head a CTA can hold
// key/value tiles in flight per CTA: enough bytes on their way per SM (two CTAs) to cover the memory's
// latency at full rate, so twice as many where a tile is half as large
__host__ __device__ constexpr int dec_stages(int dp) { return dp <= 64 ? 6 : 3; }
constexpr int PLAN_HEADER = 4;  // int32 before the first piece of a plan: [0] = number of pieces
constexpr int PLAN_ENTRY = 8;   // int32 per piece: token row, request, position, first key, first tile, tiles,
                                // pieces of the token << 16 | index of this one, rank of the token among the small ones
constexpr int PLAN_THREADS = 512;
constexpr int PLAN_SORT_MAX = 1024;   // up to this many pieces are put in order of their length, longest first
constexpr int PLAN_TOKENS_MAX = 16 * PLAN_THREADS;

// How the decode step's attention is shared out, decided once per step for all layers: with T the
// 64-key tiles of all tokens of portions of at most dec_max tokens and t = max(min_tiles,
// T * kv_heads / target_ctas) the share of one CTA, a token of n tiles is cut into max(1, n / t)
// equal pieces, whatever lengths the other requests have.  One CTA per piece and key/value head
// reads its work from the plan; nothing of the step's metadata is looked at again.
__global__ void __launch_bounds__(PLAN_THREADS)
attn_decode_plan_kernel(int* __restrict__ plan, int capacity, const int* __restrict__ positions,
                        const int* __restrict__ req_of_token, const int* __restrict__ q_start, int num_entries, int window,
                        int dec_max, int direct, int num_small, int min_tiles, int target_ctas, int nkv, int* err) {
    __shared__ int warp_sums[PLAN_THREADS / 32];
    __shared__ int piece_tiles[PLAN_SORT_MAX];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    auto block_scan = [&](int mine, int& before_me) -> int {   // exclusive prefix of `mine` over the threads; returns the total
        int incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        __syncthreads();   // the sums of an earlier scan have been read
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        before_me = incl - mine;
        int total = 0;
        for (int w = 0; w < PLAN_THREADS / 32; ++w) {
            if (w < warp) before_me += warp_sums[w];
            total += warp_sums[w];
        }
        return total;
    };
    constexpr int EACH_MAX = PLAN_TOKENS_MAX / PLAN_THREADS;
    const int each = (num_small + PLAN_THREADS - 1) / PLAN_THREADS;
    int tiles[EACH_MAX], tok[EACH_MAX], sum = 0, unused;
#pragma unroll
    for (int i = 0; i < EACH_MAX; ++i) {
        const int z = (int)threadIdx.x * each + i;
        tiles[i] = 0;
        tok[i] = -1;
        if (i < each && z < num_small) {
            const int t = small_token(z, q_start, num_entries, dec_max, direct);
            if (t >= 0 && req_of_token[t] >= 0) {
                const int pos = positions[t];
                const int lo = window > 0 ? max(0, pos - window + 1) : 0;
                tiles[i] = pos / KT - lo / KT + 1;
                tok[i] = t;
            }
        }
        sum += tiles[i];
    }
    const long long all_tiles = (long long)block_scan(sum, unused) * nkv;
    // the share as an int (a larger one would cut nothing anyway), so that the divisions below are short ones:
    // every thread of the block goes through them, most with nothing to divide
    const int share = (int)max((long long)min_tiles, min((all_tiles + target_ctas - 1) / target_ctas, (long long)INT_MAX));
    int pieces = 0, at;
#pragma unroll
    for (int i = 0; i < EACH_MAX; ++i) {
        if (tiles[i] == 0) continue;
        pieces += max(1, tiles[i] / share);
    }
    const int total = block_scan(pieces, at);
    if (threadIdx.x == 0) {
        plan[0] = total <= capacity ? total : 0;
        if (total > capacity) atomicOr(err, XB_ERR_BAD_ROW);   // the plan was sized for fewer pieces
    }
    if (total > capacity) return;
    // CTAs start in the order of the plan: the longest pieces first, so that no long one is left for the end
    const bool sorted = total <= PLAN_SORT_MAX;
    if (sorted) {
        int a = at;
#pragma unroll
        for (int i = 0; i < EACH_MAX; ++i) {
            if (!tiles[i]) continue;
            const int n = tiles[i], cz = max(1, n / share), sz = (n + cz - 1) / cz;
            for (int j = 0; j < cz; ++j, ++a) piece_tiles[a] = j * sz < n ? min(sz, n - j * sz) : 0;
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < EACH_MAX; ++i) {
        if (!tiles[i]) continue;
        const int z = (int)threadIdx.x * each + i, t = tok[i], n = tiles[i];
        const int cz = max(1, n / share);
        const int sz = (n + cz - 1) / cz, ns = (n + sz - 1) / sz;   // tiles per piece; pieces that hold any
        const int pos = positions[t];
        const int lo = window > 0 ? max(0, pos - window + 1) : 0;
        for (int j = 0; j < cz; ++j, ++at) {
            int where = at;
            if (sorted) {   // as many pieces are longer (or as long and earlier) as this one's place says
                const int mine = piece_tiles[at];
                where = 0;
                for (int o = 0; o < total; ++o) where += (piece_tiles[o] > mine || (piece_tiles[o] == mine && o < at)) ? 1 : 0;
            }
            int* e = plan + PLAN_HEADER + (size_t)where * PLAN_ENTRY;
            const int i0 = j * sz;
            e[0] = t;
            e[1] = req_of_token[t];
            e[2] = pos;
            e[3] = lo;
            e[4] = lo / KT + i0;
            e[5] = i0 < n ? min(sz, n - i0) : 0;   // an empty piece (rounding): its CTA leaves
            e[6] = (ns << 16) | j;
            e[7] = z;
        }
    }
}

// One CTA = one piece of the plan x one key/value head.  The query heads of the group are rows
// 0..G-1 of a 128-row MMA tile (rows from G on hold whatever the shared memory behind the 16-row
// query and probability tiles holds: rows never mix, and only rows below G are read back).
// Warp 0: softmax (each row's 64 scores spread over four lanes) and the epilogue.  Warps 1 and 3:
// TMA producers of keys and of values (a ring each), one lane per page box.  Warp 2: MMA issuer.
// Shared memory:
//   Q [DP/64][16 rows][64]   P[2] [16][64]   stage s: K [DP/64][64 keys][64], V likewise   barriers, pages
// Tensor memory: S[0] at column 0, S[1] at 64, O at 128.  The scores of tile i+1 are computed while
// tile i's softmax runs; P is double-buffered, so the softmax warp waits for the tensor cores only
// when a row's reference maximum has to move (then O is rescaled in TMEM).  The pieces of one token
// and head are merged by the CTA that finishes last (a ticket per token and key/value head), in
// the order of the pieces.
template <int DP>
__global__ void __launch_bounds__(128)
attn_decode_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                      float* __restrict__ part_o, float* __restrict__ part_ml, const int* __restrict__ plan,
                      const int* __restrict__ block_table, int table_stride, int nh, int nkv, int d, int ps,
                      int ps_shift, int num_pages, float scale_log2, int dec_max, int splits_max, int page_cap,
                      int* __restrict__ tickets, int* err) {
    constexpr int HALVES = DP / 64, DEC_STAGES = dec_stages(DP);
    constexpr uint32_t Q_HALF = DEC_ROWS * 128, Q_BYTES = HALVES * Q_HALF, P_ONE = DEC_ROWS * 128, P_BYTES = 2 * P_ONE;
    constexpr uint32_t KV_HALF = KT * 128, KV_BYTES = HALVES * KV_HALF, STAGE_BYTES = 2 * KV_BYTES;
    constexpr uint32_t BAR_OFF = Q_BYTES + P_BYTES + DEC_STAGES * STAGE_BYTES;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t q_sm = base, p_sm = base + Q_BYTES, kv_sm = p_sm + P_BYTES;
    unsigned char* p_ptr = smem_raw + Q_BYTES;
    // barriers, 8 bytes each: k_full k_empty v_full v_empty (one per stage each), s_ready[2] s_free[2] p_ready[2]
    // pv_done[2] q_full; then four words
    constexpr uint32_t RING_BARS = 8 * DEC_STAGES;
    const uint32_t bars = base + BAR_OFF;
    const uint32_t k_full0 = bars, k_empty0 = bars + RING_BARS, v_full0 = bars + 2 * RING_BARS, v_empty0 = bars + 3 * RING_BARS;
    const uint32_t s_ready0 = bars + 4 * RING_BARS, s_free0 = s_ready0 + 16, p_ready0 = s_ready0 + 32, pv_done0 = s_ready0 + 48,
                   q_full = s_ready0 + 64;
    volatile uint32_t* words = reinterpret_cast<volatile uint32_t*>(smem_raw + BAR_OFF + 4 * RING_BARS + 72);  // tmem, dead, last, skip
    int* s_pages = reinterpret_cast<int*>(smem_raw + BAR_OFF + 4 * RING_BARS + 96);   // this range's part of the block table
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();

    // what this CTA works on: the plan was written by the step's first kernel, before any kernel that runs
    // under programmatic dependent launch could have started
    const int G = nh / nkv, g = blockIdx.x;   // heads vary fastest: pieces start in the order of the plan
    if ((int)blockIdx.y >= plan[0]) return;
    const int4 e0 = __ldg(reinterpret_cast<const int4*>(plan + PLAN_HEADER) + 2 * blockIdx.y);
    const int4 e1 = __ldg(reinterpret_cast<const int4*>(plan + PLAN_HEADER) + 2 * blockIdx.y + 1);
    const int t = e0.x, b = e0.y, pos = e0.z, lo = e0.w, kt_first = e1.x, z = e1.w;
    const int ns = e1.z >> 16, slot = e1.z & 0xFFFF;
    if (e1.y <= 0) return;
    const int kt_last = kt_first + e1.y - 1;
    const int k_begin = max(lo, kt_first * KT), k_end = min(pos, kt_last * KT + KT - 1);
    const int fresh = pos - dec_max + 1;   // keys before this were written by earlier steps, not by the kernel before this one
    const int* table = block_table + (size_t)b * table_stride;
    const int h0 = g * G;
    const int iters = kt_last - kt_first + 1;
    const int box_rows = ps < KT ? ps : KT;
    const int page_first = (kt_first * KT) >> ps_shift;
    const int staged = min((k_end >> ps_shift) - page_first + 1, page_cap);
    for (int i = threadIdx.x; i < staged; i += 128) s_pages[i] = table[page_first + i];

    if (threadIdx.x == 0) {
        if (base & 1023u) atomicOr(err, XB_ERR_WAIT);  // the swizzle needs a 1024-byte aligned window
        words[1] = 0;
        words[2] = 0;
        words[3] = (*reinterpret_cast<volatile int*>(err) & XB_ERR_WAIT) ? 1u : 0u;   // an earlier CTA gave up: do not pile on
        for (int i = 0; i < 4 * DEC_STAGES + 2; ++i) mbar_init(bars + 8 * i, 1);   // k_full, k_empty, v_full, v_empty, s_ready
        mbar_init(s_free0, 32);
        mbar_init(s_free0 + 8, 32);
        mbar_init(p_ready0, 32);
        mbar_init(p_ready0 + 8, 32);
        mbar_init(pv_done0, 1);
        mbar_init(pv_done0 + 8, 1);
        mbar_init(q_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if ((base & 1023u) || words[3]) return;
    constexpr uint32_t TMEM_COLS = 256;
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(const_cast<uint32_t*>(&words[0]))), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = words[0];
    const uint32_t tmem_s = tmem, tmem_o = tmem + 128;

    if (warp == 1 || warp == 3) {
        // ---- producers: warp 1 streams the key pages, warp 3 the value pages, each through its own ring, one
        // lane per box (page piece x 64-column half): the lanes look their pages up and issue their copies side
        // by side.  The key ring is freed by Q K^T, the value ring two steps later by P V.
        const bool is_v = warp == 3;
        const uint32_t full0 = is_v ? v_full0 : k_full0, empty0 = is_v ? v_empty0 : k_empty0;
        const CUtensorMap* map = is_v ? &map_v : &map_k;
        const int boxes = (KT / box_rows) * HALVES;
        const int bi = lane / HALVES, hf = lane % HALVES;
        auto issue_tile = [&](int it) {
            const int s = it % DEC_STAGES, kt = kt_first + it;
            const uint32_t dst = kv_sm + s * STAGE_BYTES + (is_v ? KV_BYTES : 0u) + hf * KV_HALF + bi * box_rows * 128;
            const int j = kt * KT + bi * box_rows;
            int page = -1;
            if (lane < boxes && j <= k_end && j + box_rows - 1 >= k_begin) {
                const int idx = (j >> ps_shift) - page_first;
                page = idx < staged ? s_pages[idx] : table[j >> ps_shift];
                if (page < 0 || page >= num_pages) {
                    atomicOr(err, XB_ERR_BAD_PAGE);
                    page = -1;
                }
            }
            const uint32_t n = __popc(__ballot_sync(0xffffffffu, page >= 0));
            if (lane == 0) mbar_expect_tx(full0 + 8 * s, n * box_rows * 128);
            __syncwarp();
            if (page >= 0) tma_load_2d(dst, map, hf * 64, (page * nkv + g) * ps + (j & (ps - 1)), full0 + 8 * s);
        };
        // tiles that hold only keys of earlier steps do not depend on the kernel before this one
        int pre = 0;
        while (pre < iters && pre < DEC_STAGES && (kt_first + pre) * KT + KT - 1 < fresh) issue_tile(pre++);
        pdl_wait();
        if (!is_v && lane == 0) {
            mbar_expect_tx(q_full, HALVES * G * 128);
#pragma unroll
            for (int h2 = 0; h2 < HALVES; ++h2) tma_load_3d(q_sm + h2 * Q_HALF, &map_q, h2 * 64, h0, t, q_full);
        }
        for (int it = pre; it < iters; ++it) {
            const int s = it % DEC_STAGES;
            if (it >= DEC_STAGES && !__all_sync(0xffffffffu, mbar_wait(empty0 + 8 * s, ((it / DEC_STAGES) - 1) & 1, err))) {
                words[1] = 1;
                break;
            }
            issue_tile(it);
        }
    } else if (warp == 2) {
        // ---- MMA issuer: QK(0), then for every tile QK(next) before PV(this) ----------------------------
        if (lane == 0) {
            const uint32_t idesc_s = umma_idesc(KT, 0), idesc_o = umma_idesc(DP, 1);
            const uint64_t dq0 = umma_desc(q_sm, 16, 1024), dk0 = umma_desc(kv_sm, 16, 1024);
            const uint64_t dp0 = umma_desc(p_sm, 16, 1024), dv0 = umma_desc(kv_sm + KV_BYTES, KV_HALF, 1024);
            auto issue_qk = [&](int it) -> bool {   // S[it & 1] = Q K^T of tile `it`
                const int sb = it & 1, s = it % DEC_STAGES;
                if (!mbar_wait(k_full0 + 8 * s, (it / DEC_STAGES) & 1, err)) return false;
                if (it >= 2 && !mbar_wait(s_free0 + 8 * sb, ((it >> 1) - 1) & 1, err)) return false;  // S[sb] was read
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t dk = dk0 + (uint64_t)((s * STAGE_BYTES) >> 4);
#pragma unroll
                for (int kk = 0; kk < DP / 16; ++kk) {
                    const uint32_t off = (kk >> 2), inner = (kk & 3) * 32;
                    umma_bf16(tmem_s + (uint32_t)sb * 64, dq0 + (uint64_t)((off * Q_HALF + inner) >> 4),
                              dk + (uint64_t)((off * KV_HALF + inner) >> 4), idesc_s, kk ? 1u : 0u);
                }
                umma_commit(k_empty0 + 8 * s);   // the key stage is free once these have completed
                umma_commit(s_ready0 + 8 * sb);
                return true;
            };
            bool ok = mbar_wait(q_full, 0, err) && issue_qk(0);
            for (int it = 0; it < iters && ok; ++it) {
                const int s = it % DEC_STAGES, pb = it & 1;
                if (it + 1 < iters) ok = issue_qk(it + 1);
                ok = ok && mbar_wait(v_full0 + 8 * s, (it / DEC_STAGES) & 1, err);
                ok = ok && mbar_wait(p_ready0 + 8 * pb, (it >> 1) & 1, err);   // P written, V rows zeroed, O rescaled
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // O += P V : A = P [rows x 64 keys] K-major, B = V [64 keys x DP] MN-major (halves 64 columns apart)
                const uint64_t dp = dp0 + (uint64_t)((pb * P_ONE) >> 4);
                const uint64_t dv = dv0 + (uint64_t)((s * STAGE_BYTES) >> 4);
#pragma unroll
                for (int kk = 0; kk < KT / 16; ++kk)
                    umma_bf16(tmem_o, dp + (uint64_t)((kk * 32) >> 4), dv + (uint64_t)((kk * 2048) >> 4), idesc_o, (it | kk) ? 1u : 0u);
                umma_commit(v_empty0 + 8 * s);       // the value stage is free again once these have completed
                umma_commit(pv_done0 + 8 * pb);      // and so is P[pb]; O holds this tile
            }
            if (!ok) words[1] = 1;
        }
    } else if (warp == 0) {
        // ---- softmax: lane t works on rows t/4 and t/4 + 8, a quarter of their columns each -----------------------
        const int quad = lane & 3, r0 = lane >> 2;
        const bool two = G > 8;
        float m_ref[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
        bool alive = true;
        for (int it = 0; it < iters; ++it) {
            const int s = it & 1, key0 = (kt_first + it) * KT;
            if (!__all_sync(0xffffffffu, mbar_wait(s_ready0 + 8 * s, (it >> 1) & 1, err))) {
                alive = false;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t raw[32];
            tmem_ld_16x256b_x8(tmem_s + s * 64, raw);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(s_free0 + 8 * s);   // S[s] is in registers
            const bool edge = key0 < k_begin || key0 + KT - 1 > k_end;
            float corr[2] = {1.f, 1.f};
            int moved = 0;
            uint32_t pk[2][8];
#pragma unroll
            for (int set = 0; set < 2; ++set) {
                if (set == 1 && !two) break;
                float sc[16];
                float mx2[2] = {-INFINITY, -INFINITY};   // over the raw scores: the scale is positive
#pragma unroll
                for (int k = 0; k < 8; ++k)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        float v = __uint_as_float(raw[4 * k + 2 * set + e]);
                        if (edge) {
                            const int j = key0 + 8 * k + 2 * quad + e;
                            v = (j >= k_begin && j <= k_end) ? v : -INFINITY;
                        }
                        sc[2 * k + e] = v;
                        mx2[e] = fmaxf(mx2[e], v);
                    }
                float mx = fmaxf(mx2[0], mx2[1]);
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                mx *= scale_log2;
                // move the reference maximum only when the row's maximum outgrows it by more than 2^8
                if (mx > m_ref[set] + RESCALE_STEP) {
                    corr[set] = m_ref[set] == -INFINITY ? 0.f : ex2(m_ref[set] - mx);
                    m_ref[set] = mx;
                    moved |= (it > 0 && r0 + 8 * set < G) ? 1 : 0;
                }
                const float m_neg = m_ref[set] == -INFINITY ? 0.f : -m_ref[set];
                float sum2[2] = {0.f, 0.f};
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float e0 = ex2(fmaf(sc[2 * k], scale_log2, m_neg)), e1 = ex2(fmaf(sc[2 * k + 1], scale_log2, m_neg));
                    sum2[0] += e0;
                    sum2[1] += e1;
                    pk[set][k] = pack_bf16(e0, e1);
                }
                float sum = sum2[0] + sum2[1];
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                l[set] = l[set] * corr[set] + sum;
            }
            // P[it & 1] belongs to the P V of two tiles ago until that has completed
            if (it >= 2 && !__all_sync(0xffffffffu, mbar_wait(pv_done0 + 8 * s, ((it >> 1) - 1) & 1, err))) {
                alive = false;
                break;
            }
#pragma unroll
            for (int set = 0; set < 2; ++set) {
                if (set == 1 && !two) break;
                const int row = r0 + 8 * set;
                unsigned char* prow = p_ptr + s * P_ONE + row * 128 + quad * 4;
#pragma unroll
                for (int k = 0; k < 8; ++k) *reinterpret_cast<uint32_t*>(prow + ((k ^ (row & 7)) << 4)) = pk[set][k];
            }
            if (edge) {   // value rows outside the range become zeros (only tiles at the ends of the range)
                const int st = it % DEC_STAGES;
                mbar_wait(v_full0 + 8 * st, (it / DEC_STAGES) & 1, err);   // orders these writes after the TMA's
                unsigned char* v_ptr = smem_raw + Q_BYTES + P_BYTES + st * STAGE_BYTES + KV_BYTES;
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    const int row = lane + rr * 32, j = key0 + row;
                    if (j < k_begin || j > k_end) {
#pragma unroll
                        for (int hf = 0; hf < HALVES; ++hf) {
                            uint4* vr = reinterpret_cast<uint4*>(v_ptr + hf * KV_HALF + row * 128);
#pragma unroll
                            for (int c8 = 0; c8 < 8; ++c8) vr[c8] = make_uint4(0, 0, 0, 0);
                        }
                    }
                }
            }
            if (__any_sync(0xffffffffu, moved)) {
                // O holds every tile before this one once the last P V has completed; row = lane in this layout
                if (!__all_sync(0xffffffffu, mbar_wait(pv_done0 + 8 * (s ^ 1), ((it - 1) >> 1) & 1, err))) {
                    alive = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const float fa = __shfl_sync(0xffffffffu, corr[0], (lane & 7) * 4);
                const float fb = __shfl_sync(0xffffffffu, corr[1], (lane & 7) * 4);
                const float f = lane < 8 ? fa : (lane < 16 && two ? fb : 1.f);
#pragma unroll
                for (int c0 = 0; c0 < DP; c0 += 32) {
                    float o[32];
                    tmem_ld32(tmem_o + c0, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] *= f;
                    tmem_st32(tmem_o + c0, o);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P and zeroed V rows: visible to the MMA
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(p_ready0 + 8 * s);
        }
        // ---- O / l -> out, or this range's partial result; row = lane from here on ---------------------------------
        pdl_wait();
        if (alive) alive = mbar_wait(pv_done0 + 8 * ((iters - 1) & 1), ((iters - 1) >> 1) & 1, err);
        alive = __all_sync(0xffffffffu, alive);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float la = __shfl_sync(0xffffffffu, l[0], (lane & 7) * 4), lb = __shfl_sync(0xffffffffu, l[1], (lane & 7) * 4);
        const float ma = __shfl_sync(0xffffffffu, m_ref[0], (lane & 7) * 4), mb = __shfl_sync(0xffffffffu, m_ref[1], (lane & 7) * 4);
        if (alive) {
            const float l_row = lane < 8 ? la : lb, m_row = lane < 8 ? ma : mb;
            const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
            const bool valid = lane < G && ns <= splits_max;
            const int h = h0 + lane;
            const size_t pslot = ((size_t)z * nh + h) * splits_max + slot;   // by the token's rank among the small ones
#pragma unroll
            for (int c0 = 0; c0 < DP; c0 += 32) {
                float o[32];
                tmem_ld32(tmem_o + c0, o);   // warp-wide, whatever `valid` is
                if (!valid) continue;
                if (ns == 1) {
                    __nv_bfloat16* dst = out + ((size_t)t * nh + h) * d;
#pragma unroll
                    for (int c8 = 0; c8 < 4; ++c8) {
                        const int c = c0 + c8 * 8;
                        if (c < d) {
                            uint4 w;
                            w.x = pack_bf16(o[c8 * 8] * inv, o[c8 * 8 + 1] * inv);
                            w.y = pack_bf16(o[c8 * 8 + 2] * inv, o[c8 * 8 + 3] * inv);
                            w.z = pack_bf16(o[c8 * 8 + 4] * inv, o[c8 * 8 + 5] * inv);
                            w.w = pack_bf16(o[c8 * 8 + 6] * inv, o[c8 * 8 + 7] * inv);
                            *reinterpret_cast<uint4*>(dst + c) = w;
                        }
                    }
                } else {
                    float* dst = part_o + pslot * d;
#pragma unroll
                    for (int c4 = 0; c4 < 8; ++c4) {
                        const int c = c0 + c4 * 4;
                        if (c < d)
                            *reinterpret_cast<float4*>(dst + c) = make_float4(o[c4 * 4] * inv, o[c4 * 4 + 1] * inv, o[c4 * 4 + 2] * inv, o[c4 * 4 + 3] * inv);
                    }
                }
            }
            if (valid && ns > 1) {
                part_ml[pslot * 2] = m_row;
                part_ml[pslot * 2 + 1] = l_row;
            }
        } else {
            words[1] = 1;
        }
    }
    pdl_wait();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __threadfence();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
    if (ns == 1) return;
    if (ns > splits_max) {   // the scratch was sized for fewer pieces
        if (threadIdx.x == 0) atomicOr(err, XB_ERR_BAD_ROW);
        return;
    }
    // The CTA that finishes last among the pieces of this (token, key/value head) merges them:
    //   out[h] = sum_s w_s O_s / sum_s w_s,  w_s = L_s * 2^(M_s - max M),  in the order of the pieces.
    if (threadIdx.x == 0) {
        int* ticket = tickets + (size_t)z * nkv + g;
        const int mine = atomicAdd(ticket, 1);
        const int last = mine == ns - 1;
        words[2] = (uint32_t)last;
        if (last) *ticket = 0;   // ready for the next launch
    }
    __syncthreads();
    if (!words[2]) return;
    __threadfence();
    for (int row = warp; row < G; row += 4) {
        const int h = h0 + row;
        const size_t pbase = ((size_t)z * nh + h) * splits_max;
        if (ns <= 32) {
            // lane i holds the maximum and the sum of piece i; the pieces' rows are requested before those are
            // reduced, so that the whole merge is one trip to the L2 (the sums are formed in the order of the pieces)
            const float mi = lane < ns ? __ldcg(part_ml + (pbase + lane) * 2) : -INFINITY;
            const float li = lane < ns ? __ldcg(part_ml + (pbase + lane) * 2 + 1) : 0.f;
            const int c4 = lane * 4;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            float M = 0.f, W = 0.f, wi = 0.f;
            for (int i0 = 0; i0 < ns; i0 += 8) {
                float4 v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    v[i] = (i0 + i < ns && c4 < d) ? __ldcg(reinterpret_cast<const float4*>(part_o + (pbase + i0 + i) * d + c4))
                                                   : make_float4(0.f, 0.f, 0.f, 0.f);
                if (i0 == 0) {
                    M = warp_max(mi);
                    wi = lane < ns ? li * exp2f(mi - M) : 0.f;
                    W = warp_sum(wi);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float w = __shfl_sync(0xffffffffu, wi, (i0 + i) & 31);
                    if (i0 + i < ns) {
                        acc.x += v[i].x * w; acc.y += v[i].y * w; acc.z += v[i].z * w; acc.w += v[i].w * w;
                    }
                }
            }
            const float inv = W > 0.f ? 1.f / W : 0.f;
            if (c4 < d) {
                __nv_bfloat16* dst = out + ((size_t)t * nh + h) * d + c4;
                *reinterpret_cast<uint32_t*>(dst) = pack_bf16(acc.x * inv, acc.y * inv);
                *reinterpret_cast<uint32_t*>(dst + 2) = pack_bf16(acc.z * inv, acc.w * inv);
            }
            continue;
        }
        float mloc = -INFINITY;
        for (int i = lane; i < ns; i += 32) mloc = fmaxf(mloc, __ldcg(part_ml + (pbase + i) * 2));
        const float M = warp_max(mloc);
        float wloc = 0.f;
        for (int i = lane; i < ns; i += 32)
            wloc += __ldcg(part_ml + (pbase + i) * 2 + 1) * exp2f(__ldcg(part_ml + (pbase + i) * 2) - M);
        const float W = warp_sum(wloc);
        const float inv = W > 0.f ? 1.f / W : 0.f;
        for (int c4 = lane * 4; c4 < d; c4 += 128) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
            for (int i = 0; i < ns; ++i) {
                const float w = __ldcg(part_ml + (pbase + i) * 2 + 1) * exp2f(__ldcg(part_ml + (pbase + i) * 2) - M);
                const float4 v = __ldcg(reinterpret_cast<const float4*>(part_o + (pbase + i) * d + c4));
                acc.x += v.x * w; acc.y += v.y * w; acc.z += v.z * w; acc.w += v.w * w;
            }
            __nv_bfloat16* dst = out + ((size_t)t * nh + h) * d + c4;
            *reinterpret_cast<uint32_t*>(dst) = pack_bf16(acc.x * inv, acc.y * inv);
            *reinterpret_cast<uint32_t*>(dst + 2) = pack_bf16(acc.z * inv, acc.w * inv);
        }
    }
}

// ---- host: tensor maps ------------------------------------------------------------------------------------
// [rows, d] row-major bfloat16 (the pages of a cache) through boxes [box_rows x 64].
bool map_rows(CUtensorMap* out, const void* ptr, long long rows, int d, int box_rows) {
    return tensor_map_2d(out, ptr, rows, d, box_rows);
}
// q [T, nh, d] through boxes [box_tokens x box_heads x 64 columns].
bool map_q3(CUtensorMap* out, const void* ptr, long long T, int nh, int d, int box_heads, int box_tokens) {
    const long long dims[3] = {d, nh, T}, strides[2] = {d, (long long)nh * d};
    const int box[3] = {64, box_heads, box_tokens};
    return tensor_map_bf16(out, ptr, 3, dims, strides, box);
}

template <int DP>
int launch_prefill(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo, void* out,
                   const int* q_start, const int* start_pos, const int* table, int stride, int nh, int nkv, int d, int ps,
                   int ps_shift, int num_pages, int window, float sl2, const int* work, int ctas, int* err, cudaStream_t stream) {
    // Q of two heads, the key/value stages, the barriers' kilobyte, 4 KB of output staging per softmax warp and half
    constexpr size_t smem = 2 * (size_t)(DP / 64) * QT * 128 + PREFILL_STAGES * 2 * (size_t)(DP / 64) * KT * 128 + 1024 +
                            8 * (size_t)(DP / 64) * 4096;
    cudaFuncSetAttribute(attn_prefill_tc_kernel<DP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(attn_prefill_tc_kernel<DP>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    return xb_launch(attn_prefill_tc_kernel<DP>, dim3(ctas), dim3(PREFILL_THREADS), smem, stream, mq, mk, mv, mo,
                     (__nv_bfloat16*)out, q_start, start_pos, table, stride, nh, nkv, d, ps, ps_shift, num_pages,
                     window, sl2, work, err);
}

constexpr int DEC_PAGE_CAP = 1024;   // block-table entries of a piece that are staged in shared memory

template <int DP>
int launch_decode(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* out, float* part_o,
                  float* part_ml, const int* plan, int pieces, const int* table, int stride, int nh, int nkv, int d, int ps,
                  int ps_shift, int num_pages, float sl2, int dec_max, int splits_max, int* tickets, int overlap, int* err,
                  cudaStream_t stream) {
    constexpr size_t smem = (size_t)(DP / 64) * DEC_ROWS * 128 + 2 * DEC_ROWS * 128 + dec_stages(DP) * 2 * (size_t)(DP / 64) * KT * 128 +
                            32 * dec_stages(DP) + 96 + (size_t)DEC_PAGE_CAP * 4;
    cudaFuncSetAttribute(attn_decode_tc_kernel<DP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(attn_decode_tc_kernel<DP>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    return xb_launch_opt(overlap != 0, attn_decode_tc_kernel<DP>, dim3(nkv, pieces), dim3(128), smem, stream, mq, mk, mv,
                         (__nv_bfloat16*)out, part_o, part_ml, plan, table, stride, nh, nkv, d, ps, ps_shift, num_pages, sl2,
                         dec_max, splits_max, DEC_PAGE_CAP, tickets, err);
}

}  // namespace

// Portions of many tokens on the tensor cores: 128 queries of two query heads per work item, the items
// shared out among `ctas` CTAs (at most one per SM) by `work`, which xb_attn_prefill_work (host
// library) makes from the step's portions: [ctas + 1] offsets, then (portion, query tile, first query
// head, heads) per item, on the device.  `tokens` = rows of q.  Returns cudaErrorNotSupported (having done nothing)
// for a head size over 128 or not a multiple of 16, or a page size that is no power of two >= 8.
XB_EXPORT int xb_attn_prefill_tc(void* out, const void* q, const void* kc, const void* vc, const int* q_start,
                                 const int* start_pos, const int* table, int stride, int tokens,
                                 int nh, int nkv, int d, int ps, int num_pages, int window, float scale,
                                 const int* work, int ctas, int* err, cudaStream_t stream) {
    if (ctas <= 0) return 0;
    int shift = -1;
    for (int s = 3; s < 20; ++s)
        if ((1 << s) == ps) shift = s;
    if (d % 16 || d > 128 || d < 16 || nh % nkv || shift < 0 || !work) return (int)cudaErrorNotSupported;
    CUtensorMap mq, mk, mv, mo;   // out has the layout of q; a warp stores its 32 rows
    const long long rows = (long long)num_pages * nkv * ps;
    const int box_rows = ps < KT ? ps : KT;
    if (!map_q3(&mq, q, tokens, nh, d, 1, QT) || !map_q3(&mo, out, tokens, nh, d, 1, 32) || !map_rows(&mk, kc, rows, d, box_rows) ||
        !map_rows(&mv, vc, rows, d, box_rows))
        return (int)cudaErrorNotSupported;
    const float sl2 = scale * 1.4426950408889634f;
    if (d <= 64)
        return launch_prefill<64>(mq, mk, mv, mo, out, q_start, start_pos, table, stride, nh, nkv, d, ps, shift, num_pages, window,
                                  sl2, work, ctas, err, stream);
    return launch_prefill<128>(mq, mk, mv, mo, out, q_start, start_pos, table, stride, nh, nkv, d, ps, shift, num_pages, window,
                               sl2, work, ctas, err, stream);
}
// int32 a plan for `tokens` small tokens and `ctas` target CTAs must hold.
XB_EXPORT long long xb_attn_decode_plan_size(int tokens, int ctas, int nkv) {
    return PLAN_HEADER + (long long)PLAN_ENTRY * ((long long)tokens + ctas / (nkv > 0 ? nkv : 1) + 2);
}

// Decides how the attention of the step's small tokens (portions of at most dec_max tokens,
// `tokens` of them; direct != 0: every token of the batch is one) is shared out: pieces of about
// 1 / ctas of all keys, at least `min_keys` (a multiple of 64) each.  `plan` holds
// xb_attn_decode_plan_size(tokens, ctas, kv heads) int32.  It must run before the first kernel of
// the step that is launched with programmatic dependent launch: xb_attn_decode_tc reads the plan
// before it waits for the kernel before it.
XB_EXPORT int xb_attn_decode_plan(int* plan, const int* positions, const int* req_of_token, const int* q_start,
                                  int num_entries, int window, int dec_max, int direct, int tokens, int min_keys, int ctas,
                                  int nkv, int* err, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (tokens > PLAN_TOKENS_MAX) return (int)cudaErrorNotSupported;
    if (min_keys <= 0 || min_keys % KT || ctas <= 0 || nkv <= 0) return (int)cudaErrorInvalidValue;
    const int capacity = tokens + ctas / nkv + 2;
    attn_decode_plan_kernel<<<1, PLAN_THREADS, 0, stream>>>(plan, capacity, positions, req_of_token, q_start, num_entries, window,
                                                           dec_max, direct, tokens, min_keys / KT, ctas, nkv, err);
    return xb_launch_status();
}

// The step's small tokens on the tensor cores, shared out as `plan` says (made by
// xb_attn_decode_plan with the same tokens, ctas and kv heads, for the same window).  A token and
// head in several pieces is merged through scratch: part_o [tokens, nh, splits_max, d] float32,
// part_ml [tokens, nh, splits_max, 2] float32 and tickets [tokens * kv heads] int32, zero before the
// first launch (the kernel leaves them zero); splits_max must be at least
// min(ctas / kv heads + 1, longest context / min_keys + 1).  `q_rows` = rows of q.  `overlap` != 0
// lets the kernel start while the one before it drains; it then reads the plan before that kernel
// has finished, so the plan must have been made before the step's first kernel (else pass 0).
// Returns cudaErrorNotSupported (having done nothing) for a head size over 128 or not a multiple of
// 16, a page size that is no power of two >= 8, or more than 16 query heads per key/value head.
XB_EXPORT int xb_attn_decode_tc(void* out, float* part_o, float* part_ml, const void* q, const void* kc, const void* vc,
                                const int* plan, const int* table, int stride, int q_rows, int nh, int nkv, int d, int ps,
                                int num_pages, float scale, int dec_max, int splits_max, int tokens, int ctas, int* tickets,
                                int overlap, int* err, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    int shift = -1;
    for (int s = 3; s < 20; ++s)
        if ((1 << s) == ps) shift = s;
    if (d % 16 || d > 128 || d < 16 || nh % nkv || nh / nkv > DEC_ROWS || shift < 0 || tokens > PLAN_TOKENS_MAX)
        return (int)cudaErrorNotSupported;
    if (!plan || splits_max <= 0 || ctas <= 0) return (int)cudaErrorInvalidValue;
    if (splits_max > 1 && (!part_o || !part_ml || !tickets)) return (int)cudaErrorInvalidValue;
    CUtensorMap mq, mk, mv;
    const long long rows = (long long)num_pages * nkv * ps;
    const int box_rows = ps < KT ? ps : KT;
    if (!map_q3(&mq, q, q_rows, nh, d, nh / nkv, 1) || !map_rows(&mk, kc, rows, d, box_rows) || !map_rows(&mv, vc, rows, d, box_rows))
        return (int)cudaErrorNotSupported;
    const float sl2 = scale * 1.4426950408889634f;
    const int pieces = tokens + ctas / nkv + 2;   // the most the plan can hold
    if (d <= 64)
        return launch_decode<64>(mq, mk, mv, out, part_o, part_ml, plan, pieces, table, stride, nh, nkv, d, ps, shift, num_pages,
                                 sl2, dec_max, splits_max, tickets, overlap, err, stream);
    return launch_decode<128>(mq, mk, mv, out, part_o, part_ml, plan, pieces, table, stride, nh, nkv, d, ps, shift, num_pages,
                              sl2, dec_max, splits_max, tickets, overlap, err, stream);
}
