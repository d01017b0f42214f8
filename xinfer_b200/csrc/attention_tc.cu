// Prefill attention over the paged cache on the 5th-generation tensor cores.
//
// One CTA (128 row threads, a producer warp, an MMA issuer warp) owns 128 queries of one request's portion for one query head:
//   * a producer warp streams the request's key/value pages with TMA (cp.async.bulk.tensor,
//     128-byte swizzle, one box per page and 64-column half) into a two-stage ring guarded by
//     mbarriers; an issuer warp launches every tcgen05.mma and frees stages with tcgen05.commit;
//     the roles meet only through mbarriers;
//   * S = Q K^T (128 x 64 per key tile) accumulates in one of two tensor-memory buffers, so that the
//     next tile's scores are computed while this tile's softmax runs; each thread owns one query
//     row (TMEM lane), reads its 64 scores with tcgen05.ld, masks (causal, window, range), and runs
//     the softmax of its row entirely in registers (float32, base 2), writing P as bfloat16 into a
//     swizzled shared-memory tile;
//   * O += P V accumulates in tensor memory (V is the MN-major operand, read where TMA put it).
//     The running maximum is only moved when it grows by more than 2^8, so O is rescaled
//     (tcgen05.ld / tcgen05.st) rarely; the final O / l is exact either way.
// Value rows outside the request's visible keys are zeroed in shared memory before they are
// multiplied, so stale or poisoned pages cannot reach a result.  Every mbarrier wait is bounded
// (XB_ERR_WAIT in the error word on expiry, then the CTA frees its TMEM and leaves).
// Head sizes: multiples of 16 up to 128.  Page sizes: powers of two from 8.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace {

constexpr int QT = 128;  // queries per CTA
constexpr int KT = 64;   // keys per tile
constexpr long long WAIT_CYCLES = 400000000LL;  // about 0.2 s: a wait that long has failed
constexpr float RESCALE_STEP = 8.f;  // the row maximum moves only when it grows by more than 2^8

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err) {
    const long long t0 = clock64();
    for (;;) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (clock64() - t0 > WAIT_CYCLES) break;
    }
    atomicOr(err, XB_ERR_WAIT);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
// Shared-memory operand descriptor, 128-byte swizzle; byte offsets in 16-byte units, version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// D float32, A/B bfloat16, A K-major, M = 128, N = n; B K-major or MN-major.
__device__ __forceinline__ uint32_t umma_idesc(int n, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
          "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
          "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
          "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
          "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])),
          "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
          "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
          "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])),
          "r"(__float_as_uint(v[31]))
        : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// DP: head size padded to 64 or 128.  Shared memory (1024-byte aligned):
//   Q  [DP/64][128 rows][64]   K stage s [DP/64][64 keys][64]   V stage s likewise   P [128][64]
// every [rows][64] piece is a tile of 128-byte rows whose 16-byte chunks are XOR-ed with row & 7.
// Warps 0..3: one query row per thread (softmax).  Warp 4: TMA producer.  Warp 5: MMA issuer.
// Tensor memory: S[0] at column 0, S[1] at 64, O at 128.
template <int DP>
__global__ void __launch_bounds__(192)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                       const int* __restrict__ q_start, const int* __restrict__ start_pos, int num_entries,
                       const int* __restrict__ block_table, int table_stride, int nh, int nkv, int d, int ps,
                       int ps_shift, int num_pages, int window, float scale_log2, int dec_max, int* err) {
    constexpr int HALVES = DP / 64;
    constexpr uint32_t Q_BYTES = HALVES * QT * 128, KV_HALF = KT * 128, KV_BYTES = HALVES * KV_HALF;
    constexpr uint32_t STAGE_BYTES = 2 * KV_BYTES, P_BYTES = QT * 128;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t q_sm = base, kv_sm = base + Q_BYTES, p_sm = kv_sm + 2 * STAGE_BYTES;
    unsigned char* p_ptr = smem_raw + Q_BYTES + 2 * STAGE_BYTES;
    // barriers, 8 bytes each: full[2] empty[2] s_ready[2] s_free[2] q_full p_ready bar_o; then four words
    const uint32_t bars = p_sm + P_BYTES;
    const uint32_t full0 = bars, empty0 = bars + 16, s_ready0 = bars + 32, s_free0 = bars + 48;
    const uint32_t q_full = bars + 64, p_ready = bars + 72, bar_o = bars + 80;
    volatile uint32_t* words = reinterpret_cast<volatile uint32_t*>(p_ptr + P_BYTES + 88);  // tmem, entry, tile, dead
    const int warp = threadIdx.x >> 5;
    const int h = blockIdx.x, g = h / (nh / nkv);   // heads vary fastest: every head's longest tiles start first
    pdl_launch_dependents();
    pdl_wait();

    if (threadIdx.x == 0) {
        if (base & 1023u) atomicOr(err, XB_ERR_WAIT);  // the swizzle needs a 1024-byte aligned window
        int acc = 0, found = -1, tile = 0;
        for (int b = 0; b < num_entries; ++b) {
            const int n = q_start[b + 1] - q_start[b];
            if (n > dec_max) {
                const int nt = (n + QT - 1) / QT;
                if ((int)blockIdx.y < acc + nt) {
                    found = b;
                    tile = nt - 1 - ((int)blockIdx.y - acc);  // a portion's last (longest) tiles first
                    break;
                }
                acc += nt;
            }
        }
        if (*reinterpret_cast<volatile int*>(err) & XB_ERR_WAIT) found = -1;  // an earlier CTA gave up: do not pile on
        words[1] = (uint32_t)found;
        words[2] = (uint32_t)tile;
        words[3] = 0;
        for (int i = 0; i < 6; ++i) mbar_init(bars + 8 * i, 1);   // full, empty, s_ready
        mbar_init(s_free0, 128);
        mbar_init(s_free0 + 8, 128);
        mbar_init(q_full, 1);
        mbar_init(p_ready, 128);
        mbar_init(bar_o, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int b = (int)words[1];
    if (b < 0 || (base & 1023u)) return;
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

    const int n = q_start[b + 1] - q_start[b];
    const int row0 = (int)words[2] * QT;
    const int rows = min(QT, n - row0);
    const int t0 = q_start[b] + row0;
    const int p0 = start_pos[b] + row0;
    const int last_key = p0 + rows - 1;
    const int first_key = window > 0 ? max(0, p0 - window + 1) : 0;
    const int* table = block_table + (size_t)b * table_stride;
    const int kt_first = first_key / KT, kt_last = last_key / KT;
    const int iters = kt_last - kt_first + 1;
    const int box_rows = ps < KT ? ps : KT;

    if (warp == 4) {
        // ---- producer: Q once, then the key/value pages of every tile through the two stages ----------
        if (threadIdx.x == 128) {
            mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
            for (int hf = 0; hf < HALVES; ++hf) tma_load_3d(q_sm + hf * QT * 128, &map_q, hf * 64, h, t0, q_full);
            for (int it = 0; it < iters; ++it) {
                const int s = it & 1, kt = kt_first + it;
                if (it >= 2 && !mbar_wait(empty0 + 8 * s, ((it >> 1) - 1) & 1, err)) {
                    words[3] = 1;
                    break;
                }
                const uint32_t k_dst = kv_sm + s * STAGE_BYTES, v_dst = k_dst + KV_BYTES;
                uint32_t bytes = 0;
                int pages[KT / 8];
                for (int i = 0; i < KT / box_rows; ++i) {
                    const int j = kt * KT + i * box_rows;
                    pages[i] = -1;
                    if (j > last_key || j + box_rows - 1 < first_key) continue;
                    const int page = table[j >> ps_shift];
                    if (page < 0 || page >= num_pages) {
                        atomicOr(err, XB_ERR_BAD_PAGE);
                        continue;
                    }
                    pages[i] = page;
                    bytes += 2 * HALVES * box_rows * 128;
                }
                mbar_expect_tx(full0 + 8 * s, bytes);
                for (int i = 0; i < KT / box_rows; ++i) {
                    if (pages[i] < 0) continue;
                    const int j = kt * KT + i * box_rows;
                    const int grow = (pages[i] * nkv + g) * ps + (j & (ps - 1));
#pragma unroll
                    for (int hf = 0; hf < HALVES; ++hf) {
                        tma_load_2d(k_dst + hf * KV_HALF + i * box_rows * 128, &map_k, hf * 64, grow, full0 + 8 * s);
                        tma_load_2d(v_dst + hf * KV_HALF + i * box_rows * 128, &map_v, hf * 64, grow, full0 + 8 * s);
                    }
                }
            }
        }
    } else if (warp == 5) {
        // ---- MMA issuer: QK(0), then for every tile QK(next) before PV(this) ----------------------------
        if (threadIdx.x == 160) {
            const uint32_t idesc_s = umma_idesc(KT, 0), idesc_o = umma_idesc(DP, 1);
            // operand descriptors differ only in their start address (bits 0..13, in 16-byte units)
            const uint64_t dq0 = umma_desc(q_sm, 16, 1024), dk0 = umma_desc(kv_sm, 16, 1024);
            const uint64_t dp0 = umma_desc(p_sm, 16, 1024), dv0 = umma_desc(kv_sm + KV_BYTES, KV_HALF, 1024);
            auto issue_qk = [&](int it) -> bool {   // S[it & 1] = Q K^T of tile `it`
                const int sb = it & 1;
                if (!mbar_wait(full0 + 8 * sb, (it >> 1) & 1, err)) return false;
                if (it >= 2 && !mbar_wait(s_free0 + 8 * sb, ((it >> 1) - 1) & 1, err)) return false;  // every row of S[sb] was read
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t dk = dk0 + (uint64_t)((sb * STAGE_BYTES) >> 4);
#pragma unroll
                for (int kk = 0; kk < DP / 16; ++kk) {
                    const uint32_t off = (kk >> 2), inner = (kk & 3) * 32;
                    umma_bf16(tmem_s + (uint32_t)sb * 64, dq0 + (uint64_t)((off * QT * 128 + inner) >> 4),
                              dk + (uint64_t)((off * KV_HALF + inner) >> 4), idesc_s, kk ? 1u : 0u);
                }
                umma_commit(s_ready0 + 8 * sb);
                return true;
            };
            bool ok = mbar_wait(q_full, 0, err) && issue_qk(0);
            for (int it = 0; it < iters && ok; ++it) {
                const int s = it & 1;
                if (it + 1 < iters) ok = issue_qk(it + 1);
                ok = ok && mbar_wait(p_ready, it & 1, err);   // P written, V rows zeroed, O rescaled
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // O += P V : A = P [128 x 64 keys] K-major, B = V [64 keys x DP] MN-major (halves 64 columns apart)
                const uint64_t dv = dv0 + (uint64_t)((s * STAGE_BYTES) >> 4);
#pragma unroll
                for (int kk = 0; kk < KT / 16; ++kk)
                    umma_bf16(tmem_o, dp0 + (uint64_t)((kk * 32) >> 4), dv + (uint64_t)((kk * 2048) >> 4), idesc_o, (it | kk) ? 1u : 0u);
                umma_commit(empty0 + 8 * s);          // stage, P and O are free again once these have completed
                if (it + 1 == iters) umma_commit(bar_o);
            }
            if (!ok) words[3] = 1;
        }
    } else {
        // ---- softmax: one query row per thread ------------------------------------------------------------------
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        const int my_pos = p0 + (int)threadIdx.x;
        float m_ref = -INFINITY, l = 0.f;
        bool alive = true;
        for (int it = 0; it < iters; ++it) {
            const int s = it & 1, key0 = (kt_first + it) * KT;
            const uint32_t v_sm = kv_sm + s * STAGE_BYTES + KV_BYTES;
            // every wait's verdict is made warp-wide: tcgen05.ld / .st below need the whole warp
            if (!__all_sync(0xffffffffu, mbar_wait(s_ready0 + 8 * s, (it >> 1) & 1, err))) {
                alive = false;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float sc[64];
            {
                uint32_t ra[32], rb[32];
                tmem_ld32_nowait(tmem_s + s * 64 + lane_addr, ra);
                tmem_ld32_nowait(tmem_s + s * 64 + lane_addr + 32, rb);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    sc[i] = __uint_as_float(ra[i]);
                    sc[32 + i] = __uint_as_float(rb[i]);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(s_free0 + 8 * s);   // this row of S[s] is in registers
            const bool edge = key0 + KT - 1 > p0 || key0 + KT - 1 > last_key || key0 < first_key ||
                              (window > 0 && key0 < p0 + QT - 1 - window + 1);
            float mx = -INFINITY;
#pragma unroll
            for (int i = 0; i < 64; ++i) {
                float v = sc[i] * scale_log2;
                if (edge) {
                    const int j = key0 + i;
                    const bool ok = j <= my_pos && j <= last_key && (window <= 0 || j > my_pos - window);
                    v = ok ? v : -INFINITY;
                }
                sc[i] = v;
                mx = fmaxf(mx, v);
            }
            // move the reference maximum only when the row's maximum outgrows it by more than 2^8
            float corr = 1.f;
            int moved = 0;
            if (mx > m_ref + RESCALE_STEP) {
                corr = m_ref == -INFINITY ? 0.f : exp2f(m_ref - mx);
                m_ref = mx;
                moved = it > 0;
            }
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
            float sum = 0.f;
            uint4 pk[8];
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
                float e[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    e[i] = exp2f(sc[c8 * 8 + i] - m_use);
                    sum += e[i];
                }
                pk[c8].x = pack_bf16(e[0], e[1]);
                pk[c8].y = pack_bf16(e[2], e[3]);
                pk[c8].z = pack_bf16(e[4], e[5]);
                pk[c8].w = pack_bf16(e[6], e[7]);
            }
            l = l * corr + sum;
            // P and O belong to the previous tile's P V until it has completed
            if (it > 0 && !__all_sync(0xffffffffu, mbar_wait(empty0 + 8 * (s ^ 1), ((it - 1) >> 1) & 1, err))) {
                alive = false;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            unsigned char* prow = p_ptr + threadIdx.x * 128;
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) *reinterpret_cast<uint4*>(prow + ((c8 ^ (threadIdx.x & 7)) << 4)) = pk[c8];
            // value rows outside the visible keys become zeros (only tiles at the ends of the range)
            if (key0 < first_key || key0 + KT - 1 > last_key) {
                if (threadIdx.x < KT) {
                    mbar_wait(full0 + 8 * s, (it >> 1) & 1, err);   // already complete; orders these writes after the TMA's
                    const int j = key0 + (int)threadIdx.x;
                    if (j < first_key || j > last_key) {
#pragma unroll
                        for (int hf = 0; hf < HALVES; ++hf) {
                            uint4* vr = reinterpret_cast<uint4*>(smem_raw + (v_sm - base) + hf * KV_HALF + threadIdx.x * 128);
#pragma unroll
                            for (int c8 = 0; c8 < 8; ++c8) vr[c8] = make_uint4(0, 0, 0, 0);
                        }
                    }
                }
            }
            // rescale O where a row's reference maximum moved (rare after the first tiles); tcgen05.ld / .st
            // are warp-wide: a warp rescales when any of its rows moved, the other rows by 1
            if (__any_sync(0xffffffffu, moved)) {
                const float f = moved ? corr : 1.f;
#pragma unroll
                for (int c0 = 0; c0 < DP; c0 += 32) {
                    float o[32];
                    tmem_ld32(tmem_o + lane_addr + c0, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] *= f;
                    tmem_st32(tmem_o + lane_addr + c0, o);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P and zeroed V rows: visible to the MMA
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(p_ready);
        }
        // ---- O / l -> out -----------------------------------------------------------------------------------
        if (alive) alive = mbar_wait(bar_o, 0, err);
        alive = __all_sync(0xffffffffu, alive);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (alive) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const bool valid = (int)threadIdx.x < rows;
            __nv_bfloat16* dst = out + ((size_t)(t0 + (int)threadIdx.x) * nh + h) * d;
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
        } else {
            words[3] = 1;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host: tensor maps ------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

struct Key {
    const void* ptr;
    long long a, b, c;
    int box;
    bool operator==(const Key& o) const { return ptr == o.ptr && a == o.a && b == o.b && c == o.c && box == o.box; }
};
struct KeyHash {
    size_t operator()(const Key& k) const {
        return std::hash<const void*>()(k.ptr) ^ (size_t)(k.a * 1000003 + k.b * 10007 + k.c * 101 + k.box);
    }
};
std::unordered_map<Key, CUtensorMap, KeyHash>& cache() {
    static std::unordered_map<Key, CUtensorMap, KeyHash> c;
    return c;
}
std::mutex& cache_mutex() {
    static std::mutex m;
    return m;
}

// [rows, d] row-major bfloat16 through boxes [box_rows x 64], 128-byte swizzle.
bool map_rows(CUtensorMap* out, const void* ptr, long long rows, int d, int box_rows) {
    std::lock_guard<std::mutex> lock(cache_mutex());
    const Key key{ptr, rows, d, 0, box_rows};
    auto it = cache().find(key);
    if (it != cache().end()) {
        *out = it->second;
        return true;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t gdim[2] = {(cuuint64_t)d, (cuuint64_t)rows};
    const cuuint64_t gstr[1] = {(cuuint64_t)d * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t es[2] = {1, 1};
    CUtensorMap m;
    if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstr, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    if (cache().size() > 4096) cache().clear();
    cache()[key] = m;
    *out = m;
    return true;
}

// q [T, nh, d] through boxes [128 tokens x 1 head x 64 columns].
bool map_q3(CUtensorMap* out, const void* ptr, long long T, int nh, int d) {
    std::lock_guard<std::mutex> lock(cache_mutex());
    const Key key{ptr, T, nh, d, -1};
    auto it = cache().find(key);
    if (it != cache().end()) {
        *out = it->second;
        return true;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t gdim[3] = {(cuuint64_t)d, (cuuint64_t)nh, (cuuint64_t)T};
    const cuuint64_t gstr[2] = {(cuuint64_t)d * 2, (cuuint64_t)nh * d * 2};
    const cuuint32_t box[3] = {64, 1, (cuuint32_t)QT};
    const cuuint32_t es[3] = {1, 1, 1};
    CUtensorMap m;
    if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), gdim, gstr, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    if (cache().size() > 4096) cache().clear();
    cache()[key] = m;
    *out = m;
    return true;
}

template <int DP>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* out, const int* q_start,
           const int* start_pos, int num_entries, const int* table, int stride, int nh, int nkv, int d, int ps,
           int ps_shift, int num_pages, int window, float sl2, int dec_max, int tiles, int* err, cudaStream_t stream) {
    constexpr size_t smem = (size_t)(DP / 64) * QT * 128 + 2 * 2 * (size_t)(DP / 64) * KT * 128 + QT * 128 + 112;
    cudaFuncSetAttribute(attn_prefill_tc_kernel<DP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(attn_prefill_tc_kernel<DP>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    return xb_launch(attn_prefill_tc_kernel<DP>, dim3(nh, tiles), dim3(192), smem, stream, mq, mk, mv, (__nv_bfloat16*)out,
                     q_start, start_pos, num_entries, table, stride, nh, nkv, d, ps, ps_shift, num_pages, window, sl2,
                     dec_max, err);
}

}  // namespace

// Portions of more than dec_max tokens, 128 queries per CTA; `tiles` = sum over those portions of
// ceil(tokens / 128); `tokens` = rows of q.  Returns cudaErrorNotSupported (having done nothing)
// for a head size over 128 or not a multiple of 16, or a page size that is no power of two >= 8.
XB_EXPORT int xb_attn_prefill_tc(void* out, const void* q, const void* kc, const void* vc, const int* q_start,
                                 const int* start_pos, int num_entries, const int* table, int stride, int tokens,
                                 int nh, int nkv, int d, int ps, int num_pages, int window, float scale, int dec_max,
                                 int tiles, int* err, cudaStream_t stream) {
    if (tiles <= 0) return 0;
    int shift = -1;
    for (int s = 3; s < 20; ++s)
        if ((1 << s) == ps) shift = s;
    if (d % 16 || d > 128 || d < 16 || nh % nkv || shift < 0) return (int)cudaErrorNotSupported;
    CUtensorMap mq, mk, mv;
    const long long rows = (long long)num_pages * nkv * ps;
    const int box_rows = ps < KT ? ps : KT;
    if (!map_q3(&mq, q, tokens, nh, d) || !map_rows(&mk, kc, rows, d, box_rows) || !map_rows(&mv, vc, rows, d, box_rows))
        return (int)cudaErrorNotSupported;
    const float sl2 = scale * 1.4426950408889634f;
    if (d <= 64)
        return launch<64>(mq, mk, mv, out, q_start, start_pos, num_entries, table, stride, nh, nkv, d, ps, shift, num_pages,
                          window, sl2, dec_max, tiles, err, stream);
    return launch<128>(mq, mk, mv, out, q_start, start_pos, num_entries, table, stride, nh, nkv, d, ps, shift, num_pages,
                       window, sl2, dec_max, tiles, err, stream);
}
