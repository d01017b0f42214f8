// Matrix product for few tokens (decode): out[M, N] = x[M, K] . W[N, K]^T, bfloat16 in, float32
// accumulation, on the 5th-generation tensor cores.
//
// The product is bound by reading W once, so the kernel is built around streaming W:
//   * "swap AB": the 128 rows of a W tile are the M side of tcgen05.mma, the (padded) tokens the
//     N side, so the accumulator D[128 features, tokens] lives in tensor memory (TMEM);
//   * one thread issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of [128 x 64] W tiles and
//     [tokens x 64] x tiles into a ring of shared-memory stages guarded by mbarriers; one thread
//     issues the MMAs and releases stages with tcgen05.commit; all four warps read the accumulator
//     back with tcgen05.ld for the epilogue;
//   * K is split over the CTAs of a thread-block cluster; their partial tiles are summed through
//     distributed shared memory in rank order (deterministic, no scratch in global memory);
//   * the tile can be finished in place of a kernel of its own (EPI): the SiLU gate of a packed
//     gate/up projection (the tile holds 64 gate features and the 64 up features that belong to
//     them), or per-head q/k RMSNorm + rotary encoding + cache write of a packed q/k/v projection
//     whose heads are as wide as the tile.  The finished values are those of the separate kernels,
//     bit for bit: the sums are rounded to bfloat16 first, as the plain product would store them.
// Every wait on an mbarrier is bounded: on expiry the kernel sets XB_ERR_WAIT in the error word,
// skips the remaining work, frees its TMEM and returns.
#include "tc_common.cuh"
#include "qk_rope.cuh"

namespace {

using namespace xbtc;

constexpr int TILE_N = 128;   // W rows (output features) per CTA
constexpr int TILE_K = 64;    // K elements per stage (one 128-byte swizzle row)
constexpr int EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_QK = 2;

// What the finishing modes need.  EPI_SWIGLU: W holds the gate rows and, `up_rows` rows further,
// the up rows; out is [M, N] with N the gate's width.  EPI_QK: see qk_rope.cuh; nothing is written
// to `out`.
struct EpiArgs {
    int up_rows;
    xbqk::QkArgs qk;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float ld_cluster_f32(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    float v;
    asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote));
    return v;
}

// The sum over the cluster's ranks of element `e` of the partial tiles, in rank order.
__device__ __forceinline__ float cluster_sum(uint32_t part_addr, int e, uint32_t csize) {
    float v[8];
#pragma unroll
    for (uint32_t r = 0; r < 8; ++r) v[r] = r < csize ? ld_cluster_f32(part_addr + (uint32_t)e * 4u, r) : 0.f;
    float acc = v[0];
#pragma unroll
    for (uint32_t r = 1; r < 8; ++r) acc += v[r];
    return acc;
}

// grid: (tiles, splits); cluster (1, splits, 1).  mp: tokens padded to 16/32/64/128/256.
// Tiles: ceil(N / 128); EPI_SWIGLU: ceil(N / 64), and map_w's box is 64 rows high.
template <typename TO, int EPI>
__global__ void __launch_bounds__(128)
gemm_skinny_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      TO* __restrict__ out, int M, int N, int K, int mp, int k_per_split, int stages,
                      const EpiArgs epi, int* err) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * 16 + 1];
    __shared__ uint32_t s_tmem;
    // the dynamic window is aligned to 1024 bytes by hand (the swizzle repeats every 1024 bytes)
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t w_bytes = TILE_N * TILE_K * 2, x_bytes = (uint32_t)mp * TILE_K * 2;
    const uint32_t stage_bytes = w_bytes + x_bytes;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * (EPI == EPI_SWIGLU ? TILE_N / 2 : TILE_N);
    const int k_begin = blockIdx.y * k_per_split;
    const int k_end = min(K, k_begin + k_per_split);
    const int iters = k_end > k_begin ? (k_end - k_begin + TILE_K - 1) / TILE_K : 0;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[16]), accum = smem_u32(&bars[32]);
    const uint32_t tmem_cols = mp < 32 ? 32u : (uint32_t)mp;
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    if (threadIdx.x == 0) {
        // ---- producer: stream W and x tiles -------------------------------------------------------
        // The weights are never written by a kernel: the first ring of W tiles is requested before
        // waiting for the kernel that produces x, so that their flight overlaps its tail.
        const int pre = iters < stages ? iters : stages;
        auto load_w = [&](uint32_t dst, int k, uint32_t bar) {
            if (EPI == EPI_SWIGLU) {   // 64 gate rows, then the 64 up rows of the same features
                tma_load_2d(dst, &map_w, k, n0, bar);
                tma_load_2d(dst + w_bytes / 2, &map_w, k, epi.up_rows + n0, bar);
            } else {
                tma_load_2d(dst, &map_w, k, n0, bar);
            }
        };
        for (int it = 0; it < pre; ++it) {
            mbar_expect_tx(full0 + 8 * it, stage_bytes);
            load_w(base + it * stage_bytes, k_begin + it * TILE_K, full0 + 8 * it);
        }
        pdl_wait();
        for (int it = 0; it < pre; ++it)
            tma_load_2d(base + it * stage_bytes + w_bytes, &map_x, k_begin + it * TILE_K, 0, full0 + 8 * it);
        // stage and phase run along with `it` (it % stages, (it / stages) & 1): no division in this thread's loop
        int s = pre == stages ? 0 : pre;
        uint32_t phase = pre == stages ? 1u : 0u;
        for (int it = pre; it < iters; ++it) {
            if (!mbar_wait(empty0 + 8 * s, phase ^ 1u, err)) break;
            const uint32_t dst = base + s * stage_bytes;
            mbar_expect_tx(full0 + 8 * s, stage_bytes);
            load_w(dst, k_begin + it * TILE_K, full0 + 8 * s);
            tma_load_2d(dst + w_bytes, &map_x, k_begin + it * TILE_K, 0, full0 + 8 * s);
            if (++s == stages) {
                s = 0;
                phase ^= 1u;
            }
        }
    } else if (threadIdx.x == 32) {
        // ---- MMA issuer -------------------------------------------------------------------------------
        const uint32_t idesc = umma_idesc(mp);
        bool ok = true;
        int s = 0;
        uint32_t phase = 0;
        for (int it = 0; it < iters && ok; ++it) {
            ok = mbar_wait(full0 + 8 * s, phase, err);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a = base + s * stage_bytes;
            const uint64_t adesc = umma_desc(a), bdesc = umma_desc(a + w_bytes);
#pragma unroll
            for (int kk = 0; kk < TILE_K / 16; ++kk)   // 16 K elements = 32 bytes further along the swizzle row
                umma_bf16(tmem, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc, (it | kk) ? 1u : 0u);
            umma_commit(empty0 + 8 * s);   // the stage is free once these MMAs have read it
            if (++s == stages) {
                s = 0;
                phase ^= 1u;
            }
        }
        umma_commit(accum);                 // arrives when every MMA issued so far is complete
    }
    // ---- epilogue: all four warps ----------------------------------------------------------------------
    __syncwarp();
    const uint32_t csize = cluster_size(), crank = cluster_rank();
    // EPI_QK: groups of 8 lanes finish one token each (the tile is one head of 128).  The cluster's
    // ranks deal the tokens out among themselves; groups are counted from the last warp down, since
    // the first two warps hold the producer and the MMA issuer and join last.  What a group needs
    // beside the sums comes from the host and from constants, so it is fetched during the main loop.
    const int qk_group = 15 - (int)(threadIdx.x >> 3), qk_li = threadIdx.x & 7;
    const int qk_t = (int)crank + (int)csize * qk_group;
    xbqk::QkItem qk_item;
    if (EPI == EPI_QK) qk_item = xbqk::qk_prepare(epi.qk, qk_t < M ? qk_t : 0, (int)blockIdx.x, qk_li, qk_t < M, err);
    pdl_wait();   // nothing of the kernel before may still read what is written below
    const bool ready = mbar_wait(accum, 0, err);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int row = warp * 32 + lane;         // TMEM lane = row of D = output feature n0 + row
    const int n = n0 + row;
    float* part = reinterpret_cast<float*>(base_ptr);   // [mp][128] float32, over the (now idle) stages
    for (int c0 = 0; c0 < mp; c0 += 16) {
        float v[16];
        if (ready && iters > 0) {
            tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0.f;
        }
        if (EPI == EPI_PLAIN && csize == 1) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int m = c0 + i;
                if (m < M && n < N) out[(size_t)m * N + n] = from_f32<TO>(v[i]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) part[(c0 + i) * TILE_N + row] = v[i];
        }
    }
    if (EPI != EPI_PLAIN || csize > 1) {
        cluster_sync();   // every CTA of the cluster has written its partial tile
        const uint32_t part_addr = base;
        if (EPI == EPI_PLAIN) {
            // The tile's M x 128 sums are shared out evenly among the CTAs of the cluster; a thread asks all
            // ranks for its element at once (the loads are independent) and adds them in rank order.
            const int total = M * TILE_N;
            const int per = (total + (int)csize - 1) / (int)csize;
            const int e_end = min(total, ((int)crank + 1) * per);
            for (int e = (int)crank * per + (int)threadIdx.x; e < e_end; e += 128) {
                const float acc = cluster_sum(part_addr, e, csize);
                const int m = e / TILE_N, col = n0 + e % TILE_N;
                if (col < N) out[(size_t)m * N + col] = from_f32<TO>(acc);
            }
        } else if (EPI == EPI_SWIGLU) {
            // M x 64 gated values, shared out the same way: gate feature j sits in column j of the tile,
            // its up feature in column 64 + j
            const int total = M * (TILE_N / 2);
            const int per = (total + (int)csize - 1) / (int)csize;
            const int e_end = min(total, ((int)crank + 1) * per);
            for (int e = (int)crank * per + (int)threadIdx.x; e < e_end; e += 128) {
                const int m = e / (TILE_N / 2), j = e % (TILE_N / 2);
                const float g = bf16_round(cluster_sum(part_addr, m * TILE_N + j, csize));
                const float u = bf16_round(cluster_sum(part_addr, m * TILE_N + TILE_N / 2 + j, csize));
                const int col = n0 + j;
                if (col < N) out[(size_t)m * N + col] = from_f32<TO>(silu_mul_bf16(g, u));
            }
        } else {
            // the first pass uses what was prepared above; more than 16 tokens per rank take further passes
            for (int t0 = 0; t0 < M; t0 += (int)csize * 16) {   // the same trip count on every lane
                const int t = t0 + qk_t;
                if (t0 > 0) qk_item = xbqk::qk_prepare(epi.qk, t < M ? t : 0, (int)blockIdx.x, qk_li, t < M, err);
                float a[8], b[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    a[e] = t < M ? bf16_round(cluster_sum(part_addr, t * TILE_N + qk_li * 8 + e, csize)) : 0.f;
                    b[e] = t < M ? bf16_round(cluster_sum(part_addr, t * TILE_N + TILE_N / 2 + qk_li * 8 + e, csize)) : 0.f;
                }
                xbqk::qk_finish<8>(epi.qk, qk_item, a, b, qk_li);
            }
        }
        cluster_sync();   // nobody leaves while a neighbour still reads its shared memory
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
    }
}

// ---- host side: the launch ------------------------------------------------------------------------------
template <typename TO, int EPI>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, void* out, int M, int N, int K, int mp, int tiles, int splits,
           int k_per_split, int stages, size_t smem, const EpiArgs& epi, int* err, cudaStream_t stream) {
    cudaFuncSetAttribute(gemm_skinny_tc_kernel<TO, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles, splits, 1);
    cfg.blockDim = dim3(128, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = splits;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = xb_pdl_enabled() ? 2 : 1;
    const cudaError_t rc = cudaLaunchKernelEx(&cfg, gemm_skinny_tc_kernel<TO, EPI>, mw, mx, (TO*)out, M, N, K, mp, k_per_split, stages,
                                              epi, err);
    return rc != cudaSuccess ? (int)rc : xb_launch_status();
}

// How a product of M tokens over `tiles` tiles of W and K is laid out on the device.
struct Shape {
    int mp, splits, tiles_per_split, stages;
    size_t smem;
};

// `finished`: the tile is finished in shared memory (EPI other than plain), which needs the room
// of a float32 tile even without a cluster.
bool shape_of(Shape* sh, int M, int tiles, int K, int splits, bool finished) {
    if (M > 256 || K % 8 || K < TILE_K) return false;
    int mp = 16;
    while (mp < M) mp *= 2;
    const int k_tiles = (K + TILE_K - 1) / TILE_K;
    if (splits <= 0) {
        // enough CTAs to fill 148 SMs, at least 4 K tiles per CTA, at most 8 CTAs per cluster
        splits = 1;
        while (splits < 8 && tiles * splits < 148 && k_tiles / (splits * 2) >= 4) splits *= 2;
    }
    if (splits > 8) splits = 8;
    int tiles_per_split = (k_tiles + splits - 1) / splits;
    while (splits > 1 && (splits - 1) * tiles_per_split >= k_tiles) --splits;   // no empty split
    tiles_per_split = (k_tiles + splits - 1) / splits;
    const size_t stage_bytes = (size_t)TILE_N * TILE_K * 2 + (size_t)mp * TILE_K * 2;
    // few tokens: stages small enough for two CTAs per SM, so that a wave holds every CTA
    const size_t budget = mp <= 128 ? 100 * 1024 : 200 * 1024;
    int stages = (int)(budget / stage_bytes);
    if (stages > 12) stages = 12;
    if (stages > tiles_per_split) stages = tiles_per_split < 2 ? 2 : tiles_per_split;
    size_t smem = stages * stage_bytes;
    const size_t part = (size_t)mp * TILE_N * 4;
    if ((splits > 1 || finished) && smem < part) smem = part;
    smem += 1024;  // room to align the window to 1024 bytes
    *sh = {mp, splits, tiles_per_split, stages, smem};
    return true;
}

}  // namespace

// out[M, N] (bfloat16 when out_f32 == 0, else float32) = x[M, K] . w[N, K]^T for M <= 256.
// K must be a multiple of 8 (rows 16-byte aligned); `splits` in 1..8 CTAs share K through a
// cluster (0: chosen here).  Returns cudaErrorNotSupported for shapes it does not take.
XB_EXPORT int xb_gemm_skinny_tc(void* out, int out_f32, const void* x, const void* w, int M, int N, int K, int splits,
                                int* err, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return (int)cudaErrorNotSupported;
    const int tiles = (N + TILE_N - 1) / TILE_N;
    Shape sh;
    if (!shape_of(&sh, M, tiles, K, splits, false)) return (int)cudaErrorNotSupported;
    CUtensorMap mw, mx;
    if (!tensor_map_2d(&mw, w, N, K, TILE_N) || !tensor_map_2d(&mx, x, M, K, sh.mp)) return (int)cudaErrorNotSupported;
    const EpiArgs none = {};
    if (out_f32)
        return launch<float, EPI_PLAIN>(mw, mx, out, M, N, K, sh.mp, tiles, sh.splits, sh.tiles_per_split * TILE_K, sh.stages, sh.smem,
                                        none, err, stream);
    return launch<__nv_bfloat16, EPI_PLAIN>(mw, mx, out, M, N, K, sh.mp, tiles, sh.splits, sh.tiles_per_split * TILE_K, sh.stages,
                                            sh.smem, none, err, stream);
}

// out[M, I] = silu(x . Wg^T) * (x . Wu^T) for w = [Wg; Wu] of [2 I, K] (gate rows first), bfloat16:
// the packed gate/up projection and the SiLU gate in one kernel.  Same limits as xb_gemm_skinny_tc.
XB_EXPORT int xb_gemm_skinny_swiglu(void* out, const void* x, const void* w, int M, int I, int K, int splits, int* err,
                                    cudaStream_t stream) {
    if (M <= 0 || I <= 0) return 0;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return (int)cudaErrorNotSupported;
    const int tiles = (I + TILE_N / 2 - 1) / (TILE_N / 2);
    Shape sh;
    if (!shape_of(&sh, M, tiles, K, splits, true)) return (int)cudaErrorNotSupported;
    CUtensorMap mw, mx;
    if (!tensor_map_2d(&mw, w, 2 * I, K, TILE_N / 2) || !tensor_map_2d(&mx, x, M, K, sh.mp)) return (int)cudaErrorNotSupported;
    EpiArgs epi = {};
    epi.up_rows = I;
    return launch<__nv_bfloat16, EPI_SWIGLU>(mw, mx, out, M, I, K, sh.mp, tiles, sh.splits, sh.tiles_per_split * TILE_K, sh.stages,
                                             sh.smem, epi, err, stream);
}

// The packed q/k/v projection of M tokens, finished per head: q/k RMSNorm, rotary encoding, q to
// q_out and k/v into their cache pages (arguments as xb_qk_norm_rope_write_bf16).  Heads must be
// 128 wide (one tile of the product); other sizes get cudaErrorNotSupported and the caller runs the
// two kernels.
XB_EXPORT int xb_gemm_skinny_qkv(
    void* q_out, void* k_cache, void* v_cache, const void* x, const void* w, int M, int K, int splits, const float* q_w,
    const float* k_w, const float* cos_t, const float* sin_t, const int* positions, const int* req_of_token,
    const int* block_table, int table_stride, int nh, int nkv, int d, int rot, int interleaved, int page_size, int num_pages,
    int max_pos, float eps, int write_kv, int* err, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (d != TILE_N || (cos_t && !interleaved && rot != d) || (cos_t && (rot % 2 || rot > d))) return (int)cudaErrorNotSupported;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return (int)cudaErrorNotSupported;
    const int tiles = nh + 2 * nkv;
    const int N = tiles * TILE_N;
    Shape sh;
    if (!shape_of(&sh, M, tiles, K, splits, true)) return (int)cudaErrorNotSupported;
    CUtensorMap mw, mx;
    if (!tensor_map_2d(&mw, w, N, K, TILE_N) || !tensor_map_2d(&mx, x, M, K, sh.mp)) return (int)cudaErrorNotSupported;
    EpiArgs epi = {};
    epi.qk = {(__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, q_w, k_w, cos_t, sin_t, positions,
              req_of_token, block_table, table_stride, nh, nkv, d, rot, interleaved, page_size, num_pages, max_pos, eps, write_kv};
    return launch<__nv_bfloat16, EPI_QK>(mw, mx, nullptr, M, N, K, sh.mp, tiles, sh.splits, sh.tiles_per_split * TILE_K, sh.stages,
                                         sh.smem, epi, err, stream);
}
