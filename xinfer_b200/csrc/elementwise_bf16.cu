// bfloat16 versions of the memory-bound operations between the matrix products, with 16-byte
// accesses and one pass over the data: RMSNorm (optionally fused with the residual sum and a row
// gather), the SiLU gate, and per-head q/k RMSNorm + rotary encoding + cache write.  Arithmetic is
// float32 as in the plain kernels; these kernels need widths that are multiples of 8 elements and
// are otherwise interchangeable with them.
#include "common.cuh"

namespace {

struct alignas(16) Pack8 {
    __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const Pack8& p, float (&f)[8]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(p.v[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ Pack8 pack8(const float (&f)[8]) {
    Pack8 p;
#pragma unroll
    for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return p;
}

// ---- RMSNorm ---------------------------------------------------------------------------------------
// One block per output row; every thread keeps up to VPT 8-element vectors of the row in registers.
template <int VPT>
__global__ void rmsnorm_bf16_kernel(__nv_bfloat16* __restrict__ out, __nv_bfloat16* sum_out,
                                    const __nv_bfloat16* x, const __nv_bfloat16* branch,
                                    const int* __restrict__ rows, const float* __restrict__ w, int dim,
                                    int src_rows, float eps, float offset, int* err) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    int src = rows ? rows[r] : r;
    if (src < 0 || src >= src_rows) {
        if (threadIdx.x == 0) atomicOr(err, XB_ERR_BAD_ROW);
        src = 0;
    }
    const int nvec = dim / 8;
    const Pack8* xr = reinterpret_cast<const Pack8*>(x + (size_t)src * dim);
    const Pack8* br = branch ? reinterpret_cast<const Pack8*>(branch + (size_t)src * dim) : nullptr;
    float vals[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) {
            unpack8(xr[v], vals[i]);
            if (br) {
                float b[8];
                unpack8(br[v], b);
#pragma unroll
                for (int e = 0; e < 8; ++e) vals[i][e] = __bfloat162float(__float2bfloat16_rn(vals[i][e] + b[e]));
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += vals[i][e] * vals[i][e];
        }
    }
    const float total = block_sum(ss, scratch);
    const float inv = rsqrtf(total / (float)dim + eps);
    Pack8* o = reinterpret_cast<Pack8*>(out + (size_t)r * dim);
    Pack8* so = sum_out ? reinterpret_cast<Pack8*>(sum_out + (size_t)r * dim) : nullptr;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) {
            if (so) so[v] = pack8(vals[i]);
            const float4 w0 = reinterpret_cast<const float4*>(w)[2 * v], w1 = reinterpret_cast<const float4*>(w)[2 * v + 1];
            const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
            float y[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = vals[i][e] * inv * (offset + ww[e]);
            o[v] = pack8(y);
        }
    }
}

// ---- SiLU gate -----------------------------------------------------------------------------------------
__global__ void swiglu_bf16_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gu,
                                   int inter, size_t nvec) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nvec) return;
    const int vpr = inter / 8;
    const size_t t = i / vpr, c = i % vpr;
    const Pack8* row = reinterpret_cast<const Pack8*>(gu + t * 2 * inter);
    float g[8], u[8], y[8];
    unpack8(row[c], g);
    unpack8(row[vpr + c], u);
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = g[e] / (1.f + expf(-g[e])) * u[e];
    reinterpret_cast<Pack8*>(out + t * inter)[c] = pack8(y);
}

// ---- q/k norm + rotary + cache write -----------------------------------------------------------------
// A group of LPH lanes owns one (token, head); lane i of the group holds the 8-element vectors
// i and i + half_vecs of the head (the two halves a NeoX rotation pairs), so d = 16 * LPH' with
// LPH' <= LPH lanes active.  Interleaved layout pairs elements inside a vector instead.
template <int LPH>
__global__ void qk_norm_rope_write_bf16_kernel(
    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
    const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ q_w, const float* __restrict__ k_w,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t, const int* __restrict__ positions,
    const int* __restrict__ req_of_token, const int* __restrict__ block_table, int table_stride, int tokens,
    int nh, int nkv, int d, int rot, int interleaved, int page_size, int num_pages, int max_pos, float eps,
    int write_kv, int* err) {
    pdl_launch_dependents();
    pdl_wait();
    const int total_heads = nh + 2 * nkv;
    const int groups_per_block = blockDim.x / LPH;
    const long long item = (long long)blockIdx.x * groups_per_block + threadIdx.x / LPH;
    const int li = threadIdx.x % LPH;
    const int lanes = d / 16;                       // active lanes of the group
    const bool live = item < (long long)tokens * total_heads;
    const int t = live ? (int)(item / total_heads) : 0;
    const int h = live ? (int)(item % total_heads) : 0;
    const bool is_q = h < nh, is_k = h >= nh && h < nh + nkv;
    const bool active = live && li < lanes;
    const int pos = positions[t];
    const int half_vecs = d / 16;
    float a[8], b[8];  // vector li (first half of the head) and li + half_vecs (second half)
    const __nv_bfloat16* x = qkv + ((size_t)t * total_heads + h) * d;
    if (active) {
        unpack8(reinterpret_cast<const Pack8*>(x)[li], a);
        unpack8(reinterpret_cast<const Pack8*>(x)[li + half_vecs], b);
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = b[e] = 0.f;
    }
    // destination
    __nv_bfloat16* dst = nullptr;
    if (active) {
        if (is_q) {
            dst = q_out + ((size_t)t * nh + h) * d;
        } else if (write_kv && req_of_token[t] >= 0) {
            const int page = block_table[(size_t)req_of_token[t] * table_stride + pos / page_size];
            if (page < 0 || page >= num_pages) {
                atomicOr(err, XB_ERR_BAD_PAGE);
            } else {
                const int g = is_k ? h - nh : h - nh - nkv;
                dst = (is_k ? k_cache : v_cache) + (((size_t)page * nkv + g) * page_size + (pos % page_size)) * d;
            }
        }
    }
    // the sum of squares is reduced by every lane of the warp, whatever its head is, so that the
    // shuffles are never divergent
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += a[e] * a[e] + b[e] * b[e];
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o, LPH);
    if (is_q || is_k) {
        const float* nw = is_q ? q_w : k_w;
        if (nw && active) {
            const float inv = rsqrtf(ss / (float)d + eps);
            const float4* w4 = reinterpret_cast<const float4*>(nw);
            const float4 a0 = w4[2 * li], a1 = w4[2 * li + 1], b0 = w4[2 * (li + half_vecs)], b1 = w4[2 * (li + half_vecs) + 1];
            const float wa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float wb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                a[e] = a[e] * inv * wa[e];
                b[e] = b[e] * inv * wb[e];
            }
        }
        if (cos_t && active) {
            const int tp = pos < max_pos ? (pos < 0 ? 0 : pos) : max_pos - 1;
            const int half = rot / 2;
            const float* cr = cos_t + (size_t)tp * half;
            const float* sr = sin_t + (size_t)tp * half;
            if (!interleaved) {
                // element i of the head pairs with i + half; both lie in this lane only when
                // rot == d (vector li pairs with vector li + half_vecs); otherwise fall back per element
                if (rot == d) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const int j = li * 8 + e;
                        const float c = cr[j], s = sr[j];
                        const float x0 = a[e], x1 = b[e];
                        a[e] = x0 * c - x1 * s;
                        b[e] = x0 * s + x1 * c;
                    }
                }
            } else {
#pragma unroll
                for (int e = 0; e < 8; e += 2) {
                    const int ia = li * 8 + e, ib = (li + half_vecs) * 8 + e;  // even element indices
                    if (ia < rot) {
                        const float c = cr[ia / 2], s = sr[ia / 2], x0 = a[e], x1 = a[e + 1];
                        a[e] = x0 * c - x1 * s;
                        a[e + 1] = x0 * s + x1 * c;
                    }
                    if (ib < rot) {
                        const float c = cr[ib / 2], s = sr[ib / 2], x0 = b[e], x1 = b[e + 1];
                        b[e] = x0 * c - x1 * s;
                        b[e + 1] = x0 * s + x1 * c;
                    }
                }
            }
        }
    }
    if (dst) {
        reinterpret_cast<Pack8*>(dst)[li] = pack8(a);
        reinterpret_cast<Pack8*>(dst)[li + half_vecs] = pack8(b);
    }
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
#define XB_GO(V) return xb_launch(rmsnorm_bf16_kernel<V>, dim3(nrows), dim3(threads), 0, stream, (__nv_bfloat16*)out, (__nv_bfloat16*)sum_out, (const __nv_bfloat16*)x, (const __nv_bfloat16*)branch, rows, w, dim, src_rows, eps, offset, err)
    if (vpt <= 1) XB_GO(1);
    if (vpt <= 2) XB_GO(2);
    if (vpt <= 4) XB_GO(4);
#undef XB_GO
    return (int)cudaErrorInvalidValue;
}

XB_EXPORT int xb_swiglu_bf16(void* out, const void* gu, int tokens, int inter, cudaStream_t stream) {
    if (tokens <= 0 || inter <= 0) return 0;
    if (inter % 8) return (int)cudaErrorInvalidValue;
    const size_t nvec = (size_t)tokens * (inter / 8);
    return xb_launch(swiglu_bf16_kernel, dim3((unsigned)((nvec + 255) / 256)), dim3(256), 0, stream, (__nv_bfloat16*)out,
                     (const __nv_bfloat16*)gu, inter, nvec);
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
#define XB_GO(LPH)                                                                                               \
    return xb_launch(qk_norm_rope_write_bf16_kernel<LPH>, dim3((unsigned)((items + threads / LPH - 1) / (threads / LPH))), \
                     dim3(threads), 0, stream, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache,      \
                     (const __nv_bfloat16*)qkv, q_w, k_w, cos_t, sin_t, positions, req_of_token, block_table, table_stride,  \
                     tokens, nh, nkv, d, rot, interleaved, page_size, num_pages, max_pos, eps, write_kv, err)
    if (lanes <= 1) XB_GO(1);
    if (lanes <= 2) XB_GO(2);
    if (lanes <= 4) XB_GO(4);
    if (lanes <= 8) XB_GO(8);
    if (lanes <= 16) XB_GO(16);
    XB_GO(32);
#undef XB_GO
}
