// bfloat16 versions of the memory-bound operations between the matrix products, with 16-byte
// accesses and one pass over the data: RMSNorm (optionally fused with the residual sum and a row
// gather), the SiLU gate, and per-head q/k RMSNorm + rotary encoding + cache write.  Arithmetic is
// float32 as in the plain kernels; these kernels need widths that are multiples of 8 elements and
// are otherwise interchangeable with them.
#include "common.cuh"
#include "qk_rope.cuh"

namespace {

using xbqk::Pack8;
using xbqk::pack8;
using xbqk::unpack8;

// ---- RMSNorm ---------------------------------------------------------------------------------------
// A block works through rows blockIdx.x, blockIdx.x + gridDim.x, ...; every thread keeps up to VPT
// 8-element vectors of the row in registers, and the next row's vectors are requested before the
// current row is reduced, so that a block always has loads in flight.
template <int VPT>
__global__ void __launch_bounds__(1024) rmsnorm_bf16_kernel(__nv_bfloat16* __restrict__ out, __nv_bfloat16* sum_out,
                                    const __nv_bfloat16* x, const __nv_bfloat16* branch,
                                    const int* __restrict__ rows, const float* __restrict__ w, int dim,
                                    int nrows, int src_rows, float eps, float offset, int* err) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    const int nvec = dim / 8;
    // the weights are written by no kernel: they are fetched while the kernel before still runs
    float ww[VPT][8];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) {
            const float4 w0 = reinterpret_cast<const float4*>(w)[2 * v], w1 = reinterpret_cast<const float4*>(w)[2 * v + 1];
            ww[i][0] = w0.x, ww[i][1] = w0.y, ww[i][2] = w0.z, ww[i][3] = w0.w;
            ww[i][4] = w1.x, ww[i][5] = w1.y, ww[i][6] = w1.z, ww[i][7] = w1.w;
        }
    }
    pdl_wait();
    Pack8 rx[VPT], rb[VPT];
    auto fetch = [&](int r) {
        int src = rows ? rows[r] : r;
        if (src < 0 || src >= src_rows) {
            if (threadIdx.x == 0) atomicOr(err, XB_ERR_BAD_ROW);
            src = 0;
        }
        const Pack8* xr = reinterpret_cast<const Pack8*>(x + (size_t)src * dim);
        const Pack8* br = branch ? reinterpret_cast<const Pack8*>(branch + (size_t)src * dim) : nullptr;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * blockDim.x;
            if (v < nvec) {
                rx[i] = xr[v];
                if (br) rb[i] = br[v];
            }
        }
    };
    int r = blockIdx.x;
    if (r < nrows) fetch(r);
    while (r < nrows) {
        float vals[VPT][8];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * blockDim.x;
            if (v < nvec) {
                unpack8(rx[i], vals[i]);
                if (branch) {
                    float b[8];
                    unpack8(rb[i], b);
#pragma unroll
                    for (int e = 0; e < 8; ++e) vals[i][e] = __bfloat162float(__float2bfloat16_rn(vals[i][e] + b[e]));
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) ss += vals[i][e] * vals[i][e];
            }
        }
        const int next = r + gridDim.x;
        if (next < nrows) fetch(next);
        const float total = block_sum(ss, scratch);
        const float inv = rsqrtf(total / (float)dim + eps);
        Pack8* o = reinterpret_cast<Pack8*>(out + (size_t)r * dim);
        Pack8* so = sum_out ? reinterpret_cast<Pack8*>(sum_out + (size_t)r * dim) : nullptr;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * blockDim.x;
            if (v < nvec) {
                if (so) so[v] = pack8(vals[i]);
                float y[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) y[e] = vals[i][e] * inv * (offset + ww[i][e]);
                o[v] = pack8(y);
            }
        }
        r = next;
    }
}

// ---- SiLU gate -----------------------------------------------------------------------------------------
// grid (blocks along a row, rows); a thread takes SWIGLU_UNROLL vectors of the row, all loads first
// (one vector when there is too little work to fill the device that way).
constexpr int SWIGLU_THREADS = 128;
template <int SWIGLU_UNROLL>
__global__ void __launch_bounds__(SWIGLU_THREADS)
swiglu_bf16_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gu, int inter, int tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const int vpr = inter / 8;
    const int c0 = blockIdx.x * (SWIGLU_THREADS * SWIGLU_UNROLL) + threadIdx.x;
    for (int t = blockIdx.y; t < tokens; t += gridDim.y) {
        const Pack8* row = reinterpret_cast<const Pack8*>(gu + (size_t)t * 2 * inter);
        Pack8 pg[SWIGLU_UNROLL], pu[SWIGLU_UNROLL];
#pragma unroll
        for (int k = 0; k < SWIGLU_UNROLL; ++k) {
            const int c = c0 + k * SWIGLU_THREADS;
            if (c < vpr) {
                pg[k] = row[c];
                pu[k] = row[vpr + c];
            }
        }
#pragma unroll
        for (int k = 0; k < SWIGLU_UNROLL; ++k) {
            const int c = c0 + k * SWIGLU_THREADS;
            if (c < vpr) {
                float g[8], u[8], y[8];
                unpack8(pg[k], g);
                unpack8(pu[k], u);
#pragma unroll
                for (int e = 0; e < 8; ++e) y[e] = silu_mul_bf16(g[e], u[e]);
                reinterpret_cast<Pack8*>(out + (size_t)t * inter)[c] = pack8(y);
            }
        }
    }
}

// ---- SiLU gate over many rows -----------------------------------------------------------------------
// grid (blocks along a row, row walkers): a block takes U vectors per thread of rows blockIdx.y,
// blockIdx.y + gridDim.y, ...; the next row's vectors are requested before this row's are computed.
constexpr int SG_THREADS = 128, SG_U = 4;
__global__ void __launch_bounds__(SG_THREADS)
swiglu_rows_bf16_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gu, int inter, int tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const int vpr = inter / 8;
    const int c0 = blockIdx.x * (SG_THREADS * SG_U) + threadIdx.x;
    Pack8 pg[SG_U], pu[SG_U];
    auto fetch = [&](int t) {
        const Pack8* row = reinterpret_cast<const Pack8*>(gu + (size_t)t * 2 * inter);
#pragma unroll
        for (int k = 0; k < SG_U; ++k) {
            const int c = c0 + k * SG_THREADS;
            if (c < vpr) {
                pg[k] = row[c];
                pu[k] = row[vpr + c];
            }
        }
    };
    int t = blockIdx.y;
    if (t < tokens) fetch(t);
    while (t < tokens) {
        float y[SG_U][8];
#pragma unroll
        for (int k = 0; k < SG_U; ++k) {
            float g[8], u[8];
            unpack8(pg[k], g);
            unpack8(pu[k], u);
#pragma unroll
            for (int e = 0; e < 8; ++e) y[k][e] = silu_mul_bf16(g[e], u[e]);
        }
        const int next = t + gridDim.y;
        if (next < tokens) fetch(next);
#pragma unroll
        for (int k = 0; k < SG_U; ++k) {
            const int c = c0 + k * SG_THREADS;
            if (c < vpr) reinterpret_cast<Pack8*>(out + (size_t)t * inter)[c] = pack8(y[k]);
        }
        t = next;
    }
}

// ---- q/k norm + rotary + cache write -----------------------------------------------------------------
// A group of LPH lanes owns one (token, head); the arithmetic is that of qk_rope.cuh.  What does not
// depend on the projection (positions, pages, weights, angles) is fetched before the wait for its producer.
template <int LPH>
__global__ void qk_norm_rope_write_bf16_kernel(const xbqk::QkArgs A, const __nv_bfloat16* __restrict__ qkv, int tokens, int* err) {
    pdl_launch_dependents();
    const int total_heads = A.nh + 2 * A.nkv;
    const int groups_per_block = blockDim.x / LPH;
    const long long item = (long long)blockIdx.x * groups_per_block + threadIdx.x / LPH;
    const int li = threadIdx.x % LPH;
    const bool live = item < (long long)tokens * total_heads;
    const int t = live ? (int)(item / total_heads) : 0;
    const int h = live ? (int)(item % total_heads) : 0;
    const int half_vecs = A.d / 16;
    const bool active = live && li < half_vecs;
    const xbqk::QkItem it = xbqk::qk_prepare(A, t, h, li, live, err);
    pdl_wait();
    float a[8], b[8];  // vector li (first half of the head) and li + half_vecs (second half)
    const __nv_bfloat16* x = qkv + ((size_t)t * total_heads + h) * A.d;
    if (active) {
        unpack8(reinterpret_cast<const Pack8*>(x)[li], a);
        unpack8(reinterpret_cast<const Pack8*>(x)[li + half_vecs], b);
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = b[e] = 0.f;
    }
    xbqk::qk_finish<LPH>(A, it, a, b, li);
}

}  // namespace

XB_EXPORT int xb_rmsnorm_bf16(void* out, void* sum_out, const void* x, const void* branch, const int* rows,
                              const float* w, int nrows, int dim, int src_rows, float eps, float offset, int* err,
                              cudaStream_t stream) {
    if (nrows <= 0) return 0;
    if (dim % 8 || dim > 8 * 4 * 1024) return (int)cudaErrorInvalidValue;
    const int nvec = dim / 8;
    int threads = 32;
    while (threads < nvec && threads < 1024) threads *= 2;
    const int vpt = (nvec + threads - 1) / threads;
    // rows beyond what the device holds at once are taken by the same blocks in turn
    const int resident = 148 * (2048 / threads);
    const int blocks = nrows < resident ? nrows : resident;
#define XB_GO(V) return xb_launch(rmsnorm_bf16_kernel<V>, dim3(blocks), dim3(threads), 0, stream, (__nv_bfloat16*)out, (__nv_bfloat16*)sum_out, (const __nv_bfloat16*)x, (const __nv_bfloat16*)branch, rows, w, dim, nrows, src_rows, eps, offset, err)
    if (vpt <= 1) XB_GO(1);
    if (vpt <= 2) XB_GO(2);
    if (vpt <= 4) XB_GO(4);
#undef XB_GO
    return (int)cudaErrorInvalidValue;
}

XB_EXPORT int xb_swiglu_bf16(void* out, const void* gu, int tokens, int inter, cudaStream_t stream) {
    if (tokens <= 0 || inter <= 0) return 0;
    if (inter % 8) return (int)cudaErrorInvalidValue;
    const int vpr = inter / 8;
    const unsigned rows = (unsigned)(tokens < 65535 ? tokens : 65535);
    if ((long long)tokens * vpr >= 148LL * 2048 * 2) {
        const int per_block = SWIGLU_THREADS * 4;
        return xb_launch(swiglu_bf16_kernel<4>, dim3((unsigned)((vpr + per_block - 1) / per_block), rows), dim3(SWIGLU_THREADS), 0,
                         stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)gu, inter, tokens);
    }
    return xb_launch(swiglu_bf16_kernel<1>, dim3((unsigned)((vpr + SWIGLU_THREADS - 1) / SWIGLU_THREADS), rows), dim3(SWIGLU_THREADS), 0,
                     stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)gu, inter, tokens);
}

// The SiLU gate for many rows (a prompt portion): about eight blocks per SM stay resident and walk over
// the rows with the next row requested early; the same values as xb_swiglu_bf16.
XB_EXPORT int xb_swiglu_rows_bf16(void* out, const void* gu, int tokens, int inter, cudaStream_t stream) {
    if (tokens <= 0 || inter <= 0) return 0;
    if (inter % 8) return (int)cudaErrorNotSupported;
    const int vpr = inter / 8;
    const int per_block = SG_THREADS * SG_U;
    const unsigned bx = (unsigned)((vpr + per_block - 1) / per_block);
    // about eight blocks per SM stay resident and walk over the rows
    unsigned by = (148u * 8u + bx - 1) / bx;
    if (by > (unsigned)tokens) by = (unsigned)tokens;
    return xb_launch(swiglu_rows_bf16_kernel, dim3(bx, by), dim3(SG_THREADS), 0, stream, (__nv_bfloat16*)out,
                     (const __nv_bfloat16*)gu, inter, tokens);
}

// Needs d a multiple of 16 (at most 512) and, for the NeoX layout, rot == d.
XB_EXPORT int xb_qk_norm_rope_write_bf16(
    void* q_out, void* k_cache, void* v_cache, const void* qkv, const float* q_w, const float* k_w,
    const float* cos_t, const float* sin_t, const int* positions, const int* req_of_token, const int* block_table,
    int table_stride, int tokens, int nh, int nkv, int d, int rot, int interleaved, int page_size, int num_pages,
    int max_pos, float eps, int write_kv, int* err, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (d % 16 || d > 512 || (cos_t && !interleaved && rot != d) || (cos_t && (rot % 2 || rot > d))) return (int)cudaErrorInvalidValue;
    const int lanes = d / 16;
    const long long items = (long long)tokens * (nh + 2 * nkv);
    const int threads = 128;
    const xbqk::QkArgs A = {(__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, q_w, k_w, cos_t, sin_t,
                            positions, req_of_token, block_table, table_stride, nh, nkv, d, rot, interleaved, page_size,
                            num_pages, max_pos, eps, write_kv};
#define XB_GO(LPH)                                                                                               \
    return xb_launch(qk_norm_rope_write_bf16_kernel<LPH>, dim3((unsigned)((items + threads / LPH - 1) / (threads / LPH))), \
                     dim3(threads), 0, stream, A, (const __nv_bfloat16*)qkv, tokens, err)
    if (lanes <= 1) XB_GO(1);
    if (lanes <= 2) XB_GO(2);
    if (lanes <= 4) XB_GO(4);
    if (lanes <= 8) XB_GO(8);
    if (lanes <= 16) XB_GO(16);
    XB_GO(32);
#undef XB_GO
}
