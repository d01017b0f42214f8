// bfloat16 attention over the paged cache on tensor cores (mma.sync m16n8k16, float32 scores,
// softmax and accumulation), for head sizes that are multiples of 16 up to 256.
//
//  * attn_prefill_kernel: one CTA per (128 queries of one request's portion, query head); keys and
//    values stream through shared memory in tiles of 64 positions fetched page by page with
//    cp.async; causal mask, optional window, running softmax.
//  * attn_decode_kernel: for requests that bring only a few tokens.  One CTA per (token, key/value
//    head, range of key positions): the query heads that share the key/value head form the rows
//    of the tile, four warps take 16 keys each of every 64-key tile.  Ranges are cut at absolute
//    positions (multiples of the range length the host picks for the launch).  With more than one
//    range the CTAs write normalised partial outputs and (max, sum) to scratch memory, and the
//    CTA that finishes last for a (token, key/value head) merges them in range order.
//
// Cache layout: [num_pages, kv_heads, page_size, head_dim]; any page size.
// Keys a query at position p may see: max(0, p - window + 1) .. p  (window <= 0: from 0).
// Rows of a tile that lie outside a request's keys are zero-filled, never read from memory, so
// stale or poisoned pages cannot reach a result.
#include "attention_common.cuh"

namespace {

constexpr int KT = 64;  // key positions per shared-memory tile

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of 16-byte chunk c of row r in a [rows][DP] bf16 tile whose chunks are XOR-swizzled
// with the row, so that the 8 rows an ldmatrix reads lie in 8 different bank groups.
template <int DP>
__device__ __forceinline__ uint32_t tile_off(int r, int c) { return (uint32_t)(r * DP * 2 + ((c ^ (r & 7)) << 4)); }

// Where a CTA finds the page ids of the positions it reads: a copy in shared memory when the
// range is short enough, else the block table itself.  pages[i] is the page of positions
// (first + i) * page_size ...
struct PageView {
    const int* pages;
    int first;
};

template <int NT>
__device__ __forceinline__ PageView stage_pages(int* s_pages, int cap, const int* __restrict__ table,
                                                int page_lo, int page_hi) {
    PageView v;
    const int n = page_hi - page_lo + 1;
    if (n > cap) {
        v.pages = table;
        v.first = 0;
        return v;
    }
    for (int i = threadIdx.x; i < n; i += NT) s_pages[i] = table[page_lo + i];
    v.pages = s_pages;
    v.first = page_lo;
    return v;  // the caller synchronises before the first load
}

// Fetch rows key0 .. key0+KT-1 of key/value head g into a K tile and a V tile; rows outside
// [lo, hi] and columns beyond d are zero-filled; a page id outside the pool is flagged and its
// rows zero-filled.
template <int DP, int NT>
__device__ __forceinline__ void load_kv_tiles(uint32_t k_tile, uint32_t v_tile, const __nv_bfloat16* __restrict__ kc,
                                              const __nv_bfloat16* __restrict__ vc, PageView pv, int num_pages,
                                              int nkv, int g, int ps, int ps_shift, int d, int key0, int lo,
                                              int hi, int* err) {
    constexpr int CPR = DP / 8;     // 16-byte chunks per row
    constexpr int RPP = NT / CPR;   // rows per pass
    const int c = threadIdx.x % CPR, r0 = threadIdx.x / CPR;
    const bool col_ok = c * 8 < d;
#pragma unroll
    for (int i = 0; i < KT / RPP; ++i) {
        const int r = r0 + i * RPP;
        const int j = key0 + r;
        bool ok = col_ok && j >= lo && j <= hi;
        size_t off = 0;
        if (ok) {
            const int pi = ps_shift >= 0 ? (j >> ps_shift) : (j / ps);
            const int in = ps_shift >= 0 ? (j & (ps - 1)) : (j - pi * ps);
            const int page = pv.pages[pi - pv.first];
            if (page < 0 || page >= num_pages) {
                ok = false;
                atomicOr(err, XB_ERR_BAD_PAGE);
            } else {
                off = (((size_t)page * nkv + g) * ps + in) * d + c * 8;
            }
        }
        const uint32_t o = tile_off<DP>(r, c);
        cp_async16(k_tile + o, kc + off, ok ? 16 : 0);
        cp_async16(v_tile + o, vc + off, ok ? 16 : 0);
    }
}

// Fetch ROWS query rows (row r at qbase + r * row_stride elements while r < valid_rows).
template <int DP, int ROWS, int NT>
__device__ __forceinline__ void load_q_tile(uint32_t tile, const __nv_bfloat16* __restrict__ qbase,
                                            size_t row_stride, int valid_rows, int d) {
    constexpr int CPR = DP / 8;
    for (int idx = threadIdx.x; idx < ROWS * CPR; idx += NT) {
        const int r = idx / CPR, c = idx % CPR;
        const bool ok = r < valid_rows && c * 8 < d;
        cp_async16(tile + tile_off<DP>(r, c), ok ? qbase + r * row_stride + c * 8 : qbase, ok ? 16 : 0);
    }
}

// S[16 x NK keys] += Q[16 x DP] . K[NK x DP]^T for one warp.
template <int DP, int NK>
__device__ __forceinline__ void warp_qk(float (&s)[NK / 8][4], uint32_t q_tile, int q_row0, uint32_t k_tile, int k_row0) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int ks = 0; ks < DP / 16; ++ks) {
        uint32_t a[4];
        ldmatrix_x4(a, q_tile + tile_off<DP>(q_row0 + (lane & 15), ks * 2 + (lane >> 4)));
#pragma unroll
        for (int nb = 0; nb < NK / 16; ++nb) {
            uint32_t b[4];
            const int mid = lane >> 3;
            ldmatrix_x4(b, k_tile + tile_off<DP>(k_row0 + nb * 16 + (mid >> 1) * 8 + (lane & 7), ks * 2 + (mid & 1)));
            mma_bf16(s[nb * 2], a, b[0], b[1]);
            mma_bf16(s[nb * 2 + 1], a, b[2], b[3]);
        }
    }
}

// O[16 x DP] += P[16 x NK] . V[NK x DP] for one warp; P comes from the score accumulators.
template <int DP, int NK>
__device__ __forceinline__ void warp_pv(float (&o)[DP / 8][4], const float (&p)[NK / 8][4], uint32_t v_tile, int v_row0) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int kb = 0; kb < NK / 16; ++kb) {
        uint32_t a[4];
        a[0] = pack_bf16(p[kb * 2][0], p[kb * 2][1]);
        a[1] = pack_bf16(p[kb * 2][2], p[kb * 2][3]);
        a[2] = pack_bf16(p[kb * 2 + 1][0], p[kb * 2 + 1][1]);
        a[3] = pack_bf16(p[kb * 2 + 1][2], p[kb * 2 + 1][3]);
#pragma unroll
        for (int nb = 0; nb < DP / 16; ++nb) {
            uint32_t b[4];
            const int mid = lane >> 3;
            ldmatrix_x4_trans(b, v_tile + tile_off<DP>(v_row0 + kb * 16 + (mid & 1) * 8 + (lane & 7), nb * 2 + (mid >> 1)));
            mma_bf16(o[nb * 2], a, b[0], b[1]);
            mma_bf16(o[nb * 2 + 1], a, b[2], b[3]);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// prefill: NW warps, 16 queries each
// ------------------------------------------------------------------------------------------------
template <int DP, int NW>
__global__ void __launch_bounds__(NW * 32)
attn_prefill_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ q,
                    const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
                    const int* __restrict__ q_start, const int* __restrict__ start_pos, int num_entries,
                    const int* __restrict__ block_table, int table_stride, int nh, int nkv, int d, int ps,
                    int ps_shift, int num_pages, int window, float scale_log2, int dec_max, int page_cap, int* err) {
    constexpr int NT = NW * 32, QT = NW * 16;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ int s_entry, s_tile;
    constexpr int TILE_BYTES = KT * DP * 2;
    const uint32_t q_tile = smem_addr(smem_raw);
    const uint32_t kv_base = q_tile + QT * DP * 2;  // stages: [K0][V0][K1][V1]
    int* s_pages = reinterpret_cast<int*>(smem_raw + QT * DP * 2 + 4 * TILE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y, g = h / (nh / nkv);

    if (threadIdx.x == 0) {
        int acc = 0, found = -1, tile = 0;
        for (int b = 0; b < num_entries; ++b) {
            const int n = q_start[b + 1] - q_start[b];
            if (n > dec_max) {
                const int nt = (n + QT - 1) / QT;
                if ((int)blockIdx.x < acc + nt) {
                    found = b;
                    tile = nt - 1 - ((int)blockIdx.x - acc);  // a portion's last (longest) tiles come first
                    break;
                }
                acc += nt;
            }
        }
        s_entry = found;
        s_tile = tile;
    }
    __syncthreads();
    const int b = s_entry;
    if (b < 0) return;
    const int n = q_start[b + 1] - q_start[b];
    const int row0 = s_tile * QT;                     // first query of this tile within the portion
    const int rows = min(QT, n - row0);
    const int t0 = q_start[b] + row0;                 // its token index
    const int p0 = start_pos[b] + row0;               // its position
    const int last_key = p0 + rows - 1;               // newest key any row of the tile may see
    const int first_key = window > 0 ? max(0, p0 - window + 1) : 0;
    const int* table = block_table + (size_t)b * table_stride;
    const int kt_first = first_key / KT, kt_last = last_key / KT;
    const PageView pv = stage_pages<NT>(s_pages, page_cap, table, (kt_first * KT) / ps, last_key / ps);
    __syncthreads();

    load_q_tile<DP, QT, NT>(q_tile, q + ((size_t)t0 * nh + h) * d, (size_t)nh * d, rows, d);
    load_kv_tiles<DP, NT>(kv_base, kv_base + TILE_BYTES, kc, vc, pv, num_pages, nkv, g, ps, ps_shift, d,
                          kt_first * KT, first_key, last_key, err);
    cp_async_commit();

    float o[DP / 8][4];
#pragma unroll
    for (int i = 0; i < DP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const int pr[2] = {p0 + warp * 16 + (lane >> 2), p0 + warp * 16 + (lane >> 2) + 8};  // positions of this lane's two rows

    for (int kt = kt_first; kt <= kt_last; ++kt) {
        const int stage = (kt - kt_first) & 1;
        if (kt < kt_last) {
            const uint32_t nxt = kv_base + (stage ^ 1) * 2 * TILE_BYTES;
            load_kv_tiles<DP, NT>(nxt, nxt + TILE_BYTES, kc, vc, pv, num_pages, nkv, g, ps, ps_shift, d,
                                  (kt + 1) * KT, first_key, last_key, err);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t k_tile = kv_base + stage * 2 * TILE_BYTES, v_tile = k_tile + TILE_BYTES;
        const int key0 = kt * KT;
        // this warp's rows see nothing of the tile: keys all newer than its last row, or all older than its window
        const int w_last = p0 + warp * 16 + 15, w_first = p0 + warp * 16;
        const bool skip = key0 > w_last || (window > 0 && key0 + KT - 1 < w_first - window + 1);
        if (!skip) {
            float s[KT / 8][4];
#pragma unroll
            for (int i = 0; i < KT / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
            warp_qk<DP, KT>(s, q_tile, warp * 16, k_tile, 0);
            // masks are needed only where the tile touches the diagonal, the window's edge or the end
            const bool need_mask = key0 + KT - 1 > w_first || key0 + KT - 1 > last_key ||
                                   (window > 0 && key0 < w_last - window + 1);
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < KT / 8; ++i) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = s[i][e] * scale_log2;
                    if (need_mask) {
                        const int j = key0 + i * 8 + (lane & 3) * 2 + (e & 1);
                        const int p = pr[e >> 1];
                        const bool ok = j <= p && j <= last_key && (window <= 0 || j > p - window);
                        v = ok ? v : -INFINITY;
                    }
                    s[i][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m[r], mx[r]);
                const float m_use = m_new == -INFINITY ? 0.f : m_new;
                const float corr = exp2f(m[r] - m_use);
                m[r] = m_new;
                l[r] *= corr;
#pragma unroll
                for (int i = 0; i < DP / 8; ++i) {
                    o[i][r * 2] *= corr;
                    o[i][r * 2 + 1] *= corr;
                }
                float sum = 0.f;
#pragma unroll
                for (int i = 0; i < KT / 8; ++i) {
                    const float a = exp2f(s[i][r * 2] - m_use), c = exp2f(s[i][r * 2 + 1] - m_use);
                    s[i][r * 2] = a;
                    s[i][r * 2 + 1] = c;
                    sum += a + c;
                }
                l[r] += sum;
            }
            warp_pv<DP, KT>(o, s, v_tile, 0);
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        const int row = warp * 16 + (lane >> 2) + r * 8;
        if (row >= rows) continue;
        const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
        __nv_bfloat16* dst = out + ((size_t)(t0 + row) * nh + h) * d;
#pragma unroll
        for (int i = 0; i < DP / 8; ++i) {
            const int c = i * 8 + (lane & 3) * 2;
            if (c < d) *reinterpret_cast<uint32_t*>(dst + c) = pack_bf16(o[i][r * 2] * inv, o[i][r * 2 + 1] * inv);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// decode (few tokens per request), split over key ranges
// ------------------------------------------------------------------------------------------------
template <int DP>
__global__ void __launch_bounds__(128)
attn_decode_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                   const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                   const __nv_bfloat16* __restrict__ vc, const int* __restrict__ positions,
                   const int* __restrict__ req_of_token, const int* __restrict__ q_start, int num_entries,
                   const int* __restrict__ block_table, int table_stride, int nh, int nkv, int d, int ps,
                   int ps_shift, int num_pages, int window, float scale_log2, int dec_max, int direct, int split,
                   int num_splits, int page_cap, int* __restrict__ tickets, int* err) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int NT = 128;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ float s_m[4][16], s_l[4][16];
    constexpr int TILE_BYTES = KT * DP * 2;
    constexpr int KV_BYTES = 4 * TILE_BYTES, MERGE_BYTES = 4 * 16 * DP * 4;
    const uint32_t q_tile = smem_addr(smem_raw);
    const uint32_t kv_base = q_tile + 16 * DP * 2;
    float* o_all = reinterpret_cast<float*>(smem_raw + 16 * DP * 2);  // reused after the loop: [4][16][DP]
    int* s_pages = reinterpret_cast<int*>(smem_raw + 16 * DP * 2 + (KV_BYTES > MERGE_BYTES ? KV_BYTES : MERGE_BYTES));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = nh / nkv;
    const int qtiles = (G + 15) / 16;
    const int g = blockIdx.y / qtiles, qt = blockIdx.y % qtiles;
    const int t = small_token(blockIdx.z, q_start, num_entries, dec_max, direct);
    if (t < 0) return;
    const int b = req_of_token[t];
    if (b < 0) return;
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int k_begin = max(lo, (int)blockIdx.x * split), k_end = min(pos, ((int)blockIdx.x + 1) * split - 1);
    if (k_begin > k_end) return;
    const int* table = block_table + (size_t)b * table_stride;
    const int h0 = g * G + qt * 16;
    const int rows = min(16, G - qt * 16);
    const int kt_first = k_begin / KT, kt_last = k_end / KT;
    const PageView pv = stage_pages<NT>(s_pages, page_cap, table, (kt_first * KT) / ps, k_end / ps);
    __syncthreads();

    load_q_tile<DP, 16, NT>(q_tile, q + ((size_t)t * nh + h0) * d, (size_t)d, rows, d);
    load_kv_tiles<DP, NT>(kv_base, kv_base + TILE_BYTES, kc, vc, pv, num_pages, nkv, g, ps, ps_shift, d,
                          kt_first * KT, k_begin, k_end, err);
    cp_async_commit();

    float o[DP / 8][4];
#pragma unroll
    for (int i = 0; i < DP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int kt = kt_first; kt <= kt_last; ++kt) {
        const int stage = (kt - kt_first) & 1;
        if (kt < kt_last) {
            const uint32_t nxt = kv_base + (stage ^ 1) * 2 * TILE_BYTES;
            load_kv_tiles<DP, NT>(nxt, nxt + TILE_BYTES, kc, vc, pv, num_pages, nkv, g, ps, ps_shift, d,
                                  (kt + 1) * KT, k_begin, k_end, err);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t k_tile = kv_base + stage * 2 * TILE_BYTES, v_tile = k_tile + TILE_BYTES;
        const int key0 = kt * KT + warp * 16;  // this warp's 16 keys of the tile
        if (key0 <= k_end && key0 + 15 >= k_begin) {
            float s[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
            warp_qk<DP, 16>(s, q_tile, 0, k_tile, warp * 16);
            // every row of the tile is the same token: one key range for all rows
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = key0 + i * 8 + (lane & 3) * 2 + (e & 1);
                    s[i][e] = (j >= k_begin && j <= k_end) ? s[i][e] * scale_log2 : -INFINITY;
                }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float mx = fmaxf(fmaxf(s[0][r * 2], s[0][r * 2 + 1]), fmaxf(s[1][r * 2], s[1][r * 2 + 1]));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m[r], mx);
                const float m_use = m_new == -INFINITY ? 0.f : m_new;
                const float corr = exp2f(m[r] - m_use);
                m[r] = m_new;
                l[r] *= corr;
#pragma unroll
                for (int i = 0; i < DP / 8; ++i) {
                    o[i][r * 2] *= corr;
                    o[i][r * 2 + 1] *= corr;
                }
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const float a = exp2f(s[i][r * 2] - m_use), c = exp2f(s[i][r * 2 + 1] - m_use);
                    s[i][r * 2] = a;
                    s[i][r * 2 + 1] = c;
                    l[r] += a + c;
                }
            }
            warp_pv<DP, 16>(o, s, v_tile, warp * 16);
        }
        __syncthreads();
    }
    // merge the four warps (each saw its own keys)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        const int row = (lane >> 2) + r * 8;
        if ((lane & 3) == 0) {
            s_m[warp][row] = m[r];
            s_l[warp][row] = l[r];
        }
        if (row < rows) {
#pragma unroll
            for (int i = 0; i < DP / 8; ++i) {
                const int c = i * 8 + (lane & 3) * 2;
                float* dst = o_all + ((size_t)warp * 16 + row) * DP + c;
                dst[0] = o[i][r * 2];
                dst[1] = o[i][r * 2 + 1];
            }
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < rows * d; idx += NT) {
        const int row = idx / d, c = idx % d;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, s_m[w][row]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = s_m[w][row] == -INFINITY ? 0.f : exp2f(s_m[w][row] - M);
            L += s_l[w][row] * f;
            O += o_all[((size_t)w * 16 + row) * DP + c] * f;
        }
        const float val = L > 0.f ? O / L : 0.f;
        const int h = h0 + row;
        if (num_splits == 1) {
            out[((size_t)t * nh + h) * d + c] = __float2bfloat16_rn(val);
        } else {
            const size_t slot = ((size_t)blockIdx.z * nh + h) * num_splits + blockIdx.x;  // by the token's rank among the small ones
            part_o[slot * d + c] = val;
            if (c == 0) {
                part_ml[slot * 2] = M;
                part_ml[slot * 2 + 1] = L;
            }
        }
    }
    if (num_splits == 1) return;
    // The CTA that finishes last among the ranges of this (token, key/value head) merges them:
    //   out[h] = sum_s w_s O_s / sum_s w_s,  w_s = L_s * 2^(M_s - max M),  in range order.
    __shared__ int s_last;
    const int s0 = lo / split, s1 = pos / split;   // the ranges this token's keys touch
    const int ns = s1 - s0 + 1;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* ticket = tickets + (size_t)blockIdx.z * gridDim.y + blockIdx.y;
        const int mine = atomicAdd(ticket, 1);
        s_last = mine == ns - 1;
        if (s_last) *ticket = 0;   // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int row = warp; row < rows; row += 4) {
        const int h = h0 + row;
        const size_t base = ((size_t)blockIdx.z * nh + h) * num_splits + s0;
        float mloc = -INFINITY;
        for (int i = lane; i < ns; i += 32) mloc = fmaxf(mloc, __ldcg(part_ml + (base + i) * 2));
        const float M = warp_max(mloc);
        float wloc = 0.f;
        for (int i = lane; i < ns; i += 32)
            wloc += __ldcg(part_ml + (base + i) * 2 + 1) * exp2f(__ldcg(part_ml + (base + i) * 2) - M);
        const float W = warp_sum(wloc);
        const float inv = W > 0.f ? 1.f / W : 0.f;
        for (int c4 = lane * 4; c4 < d; c4 += 128) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
            for (int i = 0; i < ns; ++i) {
                const float w = __ldcg(part_ml + (base + i) * 2 + 1) * exp2f(__ldcg(part_ml + (base + i) * 2) - M);
                const float4 v = __ldcg(reinterpret_cast<const float4*>(part_o + (base + i) * d + c4));
                acc.x += v.x * w; acc.y += v.y * w; acc.z += v.z * w; acc.w += v.w * w;
            }
            __nv_bfloat16* dst = out + ((size_t)t * nh + h) * d + c4;
            *reinterpret_cast<uint32_t*>(dst) = pack_bf16(acc.x * inv, acc.y * inv);
            *reinterpret_cast<uint32_t*>(dst + 2) = pack_bf16(acc.z * inv, acc.w * inv);
        }
    }
}

int shift_of(int ps) {
    for (int s = 0; s < 31; ++s)
        if ((1 << s) == ps) return s;
    return -1;
}

constexpr int PAGE_CAP_MAX = 8192;  // page ids a CTA may stage in shared memory (32 KB)

template <int DP, int NW>
int launch_prefill(void* out, const void* q, const void* kc, const void* vc, const int* q_start, const int* start_pos,
                   int num_entries, const int* table, int stride, int nh, int nkv, int d, int ps, int num_pages,
                   int window, float scale_log2, int dec_max, int tiles, int max_context, int* err, cudaStream_t stream) {
    int page_cap = (max_context + ps - 1) / ps + 2;
    if (page_cap > PAGE_CAP_MAX) page_cap = 0;
    const size_t smem = (size_t)NW * 16 * DP * 2 + 4 * KT * DP * 2 + (size_t)page_cap * 4;
    cudaFuncSetAttribute(attn_prefill_kernel<DP, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(attn_prefill_kernel<DP, NW>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    attn_prefill_kernel<DP, NW><<<dim3(tiles, nh), NW * 32, smem, stream>>>(
        (__nv_bfloat16*)out, (const __nv_bfloat16*)q, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, q_start,
        start_pos, num_entries, table, stride, nh, nkv, d, ps, shift_of(ps), num_pages, window, scale_log2, dec_max,
        page_cap, err);
    return xb_launch_status();
}

template <int DP>
int launch_decode(void* out, float* part_o, float* part_ml, const void* q, const void* kc, const void* vc,
                  const int* positions, const int* req_of_token, const int* q_start, int num_entries, const int* table,
                  int stride, int nh, int nkv, int d, int ps, int num_pages, int window, float scale_log2, int dec_max,
                  int direct, int split, int num_splits, int tokens, int* tickets, int* err, cudaStream_t stream) {
    const size_t kv = 4 * (size_t)KT * DP * 2, merge = 4 * 16 * (size_t)DP * 4;
    int page_cap = (split + KT) / ps + 2;
    if (page_cap > PAGE_CAP_MAX) page_cap = 0;
    const size_t smem = 16 * DP * 2 + (kv > merge ? kv : merge) + (size_t)page_cap * 4;
    cudaFuncSetAttribute(attn_decode_kernel<DP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(attn_decode_kernel<DP>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    const int qtiles = (nh / nkv + 15) / 16;
    return xb_launch(attn_decode_kernel<DP>, dim3(num_splits, nkv * qtiles, tokens), dim3(128), smem, stream,
                     (__nv_bfloat16*)out, part_o, part_ml, (const __nv_bfloat16*)q, (const __nv_bfloat16*)kc,
                     (const __nv_bfloat16*)vc, positions, req_of_token, q_start, num_entries, table, stride, nh, nkv, d, ps,
                     shift_of(ps), num_pages, window, scale_log2, dec_max, direct, split, num_splits, page_cap, tickets, err);
}

}  // namespace

// Portions of more than dec_max tokens, `warps` * 16 queries per CTA (warps = 4 or 8); `tiles` =
// sum over those portions of ceil(tokens / (warps * 16)); max_context = the longest
// start + tokens among them.
XB_EXPORT int xb_attn_prefill_bf16(void* out, const void* q, const void* kc, const void* vc, const int* q_start,
                                   const int* start_pos, int num_entries, const int* table, int stride, int nh,
                                   int nkv, int d, int ps, int num_pages, int window, float scale, int dec_max,
                                   int tiles, int max_context, int warps, int* err, cudaStream_t stream) {
    if (tiles <= 0) return 0;
    if (d % 16 || d > 256 || nh % nkv || ps <= 0 || (warps != 4 && warps != 8)) return (int)cudaErrorInvalidValue;
    const float sl2 = scale * 1.4426950408889634f;
#define XB_GO(DP, NW) return launch_prefill<DP, NW>(out, q, kc, vc, q_start, start_pos, num_entries, table, stride, nh, nkv, d, ps, num_pages, window, sl2, dec_max, tiles, max_context, err, stream)
    if (warps == 4) {
        if (d <= 64) XB_GO(64, 4);
        if (d <= 128) XB_GO(128, 4);
        XB_GO(256, 4);
    }
    if (d <= 64) XB_GO(64, 8);
    if (d <= 128) XB_GO(128, 8);
    XB_GO(256, 4);  // 8 warps of a 256-wide head would not fit shared memory
#undef XB_GO
}

// Tokens of portions of at most dec_max tokens (`tokens` of them; direct != 0: every token of the
// batch is one).  Keys are cut into ranges of `split` positions (a multiple of 64) at absolute
// positions; num_splits = ceil(longest context / split).  Scratch, needed when num_splits > 1:
// part_o [tokens, nh, num_splits, d] float32, part_ml [tokens, nh, num_splits, 2] float32 and
// tickets [tokens * kv heads * ceil(group / 16)] int32, zero before the first launch (the kernel
// leaves them zero).
XB_EXPORT int xb_attn_decode_bf16(void* out, float* part_o, float* part_ml, const void* q, const void* kc,
                                  const void* vc, const int* positions, const int* req_of_token, const int* q_start,
                                  int num_entries, const int* table, int stride, int nh, int nkv, int d, int ps,
                                  int num_pages, int window, float scale, int dec_max, int direct, int split,
                                  int num_splits, int tokens, int* tickets, int* err, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (d % 16 || d > 256 || nh % nkv || num_splits < 1 || split < KT || split % KT || ps <= 0) return (int)cudaErrorInvalidValue;
    if (num_splits > 1 && (!part_o || !part_ml || !tickets)) return (int)cudaErrorInvalidValue;
    const float sl2 = scale * 1.4426950408889634f;
    int rc;
#define XB_GO(DP) rc = launch_decode<DP>(out, part_o, part_ml, q, kc, vc, positions, req_of_token, q_start, num_entries, table, stride, nh, nkv, d, ps, num_pages, window, sl2, dec_max, direct, split, num_splits, tokens, tickets, err, stream)
    if (d <= 64) XB_GO(64);
    else if (d <= 128) XB_GO(128);
    else XB_GO(256);
#undef XB_GO
    return rc;
}

// ------------------------------------------------------------------------------------------------
// The same decode attention for callers that cannot allocate (see no_alloc.h): the scratch that
// xb_attn_decode_bf16 takes from its caller lives in a fixed device array of this module.
// ------------------------------------------------------------------------------------------------
#include <atomic>

#include "no_alloc.h"

namespace {
// Device memory that belongs to the loaded module.  In host code this name is only a handle for
// cudaGetSymbolAddress, never an address a kernel may be given.
static __device__ __align__(256) unsigned char xb_noalloc_scratch[XB_NOALLOC_SCRATCH_BYTES];

constexpr int NOALLOC_MAX_DEVICES = 64;
// the array's address per device; two host threads that make a device's first call together both
// look it up and store the same value
std::atomic<unsigned char*> g_noalloc_base[NOALLOC_MAX_DEVICES];

size_t noalloc_align(size_t n) { return (n + 255) & ~(size_t)255; }
}  // namespace

// Bytes of the built-in array a call with these sizes would use (tickets, (max, sum) pairs, partials).
XB_EXPORT long long xb_attn_decode_bf16_noalloc_need(int nh, int nkv, int d, int num_splits, int tokens) {
    if (num_splits <= 1 || tokens <= 0 || nkv <= 0) return 0;
    const size_t pairs = (size_t)tokens * nkv * ((nh / nkv + 15) / 16);
    const size_t slots = (size_t)tokens * nh * num_splits;
    return (long long)(noalloc_align(pairs * sizeof(int)) + noalloc_align(slots * 2 * sizeof(float)) + slots * d * sizeof(float));
}

XB_EXPORT int xb_attn_decode_bf16_noalloc(void* out, const void* q, const void* kc, const void* vc, const int* positions,
                                          const int* req_of_token, const int* q_start, int num_entries,
                                          const int* table, int stride, int nh, int nkv, int d, int ps, int num_pages,
                                          int window, float scale, int dec_max, int direct, int split, int num_splits,
                                          int tokens, int* err, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (nkv <= 0 || nh % nkv) return (int)cudaErrorInvalidValue;
    if ((size_t)xb_attn_decode_bf16_noalloc_need(nh, nkv, d, num_splits, tokens) > (size_t)XB_NOALLOC_SCRATCH_BYTES)
        return XB_NOALLOC_TOO_LARGE;
    // the array's address on the current device, looked up once per device
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return XB_NOALLOC_NO_SYMBOL;
    unsigned char* base = g_noalloc_base[dev].load(std::memory_order_acquire);
    if (!base) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, xb_noalloc_scratch) != cudaSuccess || !p) return XB_NOALLOC_NO_SYMBOL;
        base = static_cast<unsigned char*>(p);
        g_noalloc_base[dev].store(base, std::memory_order_release);
    }
    int* tickets = nullptr;
    float *part_ml = nullptr, *part_o = nullptr;
    if (num_splits > 1) {
        const size_t pairs = (size_t)tokens * nkv * ((nh / nkv + 15) / 16);
        const size_t slots = (size_t)tokens * nh * num_splits;
        tickets = reinterpret_cast<int*>(base);
        part_ml = reinterpret_cast<float*>(base + noalloc_align(pairs * sizeof(int)));
        part_o = reinterpret_cast<float*>(base + noalloc_align(pairs * sizeof(int)) + noalloc_align(slots * 2 * sizeof(float)));
        // the tickets must start at zero whatever an earlier (perhaps failed) call left behind
        const cudaError_t rc = cudaMemsetAsync(tickets, 0, pairs * sizeof(int), stream);
        if (rc != cudaSuccess) return (int)rc;
    }
    return xb_attn_decode_bf16(out, part_o, part_ml, q, kc, vc, positions, req_of_token, q_start, num_entries, table,
                               stride, nh, nkv, d, ps, num_pages, window, scale, dec_max, direct, split, num_splits,
                               tokens, tickets, err, stream);
}
