// Plain kernels for every operation of a decoder step, templated on the storage type.
//
// They are the whole float32 path (all arithmetic in float32, no tensor-core mode of reduced
// precision) and the fall-back of the bfloat16 path for sizes the tiled kernels refuse.  Each
// output element is reduced in an order that depends only on that element (its row, its key
// range), never on what else is in the batch, so float32 results are bit-identical however the
// tokens were cut into steps.
#include "common.cuh"

// ------------------------------------------------------------------------------------------
// Embedding gather: out[t, :] = table[ids[t], :].  An id -1 - i stands for sampled[i], the id a
// sampler left on the device (the host has not seen it yet).
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void embedding_kernel(T* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                                 const int* __restrict__ sampled, int num_sampled, int hidden, int vocab, float scale,
                                 int* err) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 && sampled != nullptr && -1 - id < num_sampled) id = sampled[-1 - id];
    T* o = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(err, XB_ERR_BAD_TOKEN);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<T>(0.f);
        return;
    }
    const T* r = table + (size_t)id * hidden;
    if (scale != 1.f) {   // row times a constant, the product rounded to the activation type
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<T>(to_f32<T>(r[i]) * scale);
    } else if ((hidden * sizeof(T)) % 16 == 0) {
        const int n16 = hidden * sizeof(T) / 16;
        const uint4* r4 = reinterpret_cast<const uint4*>(r);
        uint4* o4 = reinterpret_cast<uint4*>(o);
        for (int i = threadIdx.x; i < n16; i += blockDim.x) o4[i] = r4[i];
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = r[i];
    }
}

XB_EXPORT int xb_embedding(int dtype, void* out, const void* table, const int* ids, const int* sampled, int num_sampled,
                           int tokens, int hidden, int vocab, float scale, int* err, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (dtype == XB_F32)
        return xb_launch(embedding_kernel<float>, dim3(tokens), dim3(256), 0, stream, (float*)out, (const float*)table, ids,
                         sampled, num_sampled, hidden, vocab, scale, err);
    return xb_launch(embedding_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, (__nv_bfloat16*)out,
                     (const __nv_bfloat16*)table, ids, sampled, num_sampled, hidden, vocab, scale, err);
}

// ------------------------------------------------------------------------------------------
// What a model may do to its float32 logits after the head: v *= scale, then v = cap * tanh(v / cap)
// (cap <= 0: no cap).  In place.
// ------------------------------------------------------------------------------------------
__global__ void logits_post_kernel(float* __restrict__ logits, size_t n, float scale, float cap) {
    const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float v = logits[i] * scale;
        if (cap > 0.f) v = cap * tanhf(v * inv_cap);
        logits[i] = v;
    }
}

XB_EXPORT int xb_logits_post(float* logits, long long n, float scale, float cap, cudaStream_t stream) {
    if (n <= 0) return 0;
    const long long blocks = (n + 255) / 256;
    logits_post_kernel<<<(unsigned)(blocks < 4096 ? blocks : 4096), 256, 0, stream>>>(logits, (size_t)n, scale, cap);
    return xb_launch_status();
}

// ------------------------------------------------------------------------------------------
// RMSNorm, optionally preceded by the residual sum and/or a row gather.
//   s    = rows ? x[rows[r]] : x[r]            (+ branch at the same row, rounded to T)
//   out  = s * rsqrt(mean(s^2) + eps) * (offset + w)
// `sum_out` (nullable) receives s; it may alias x when no gather is asked for.
// Statistics, the weight product and the residual sum are float32.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void rmsnorm_kernel(T* __restrict__ out, T* sum_out, const T* x, const T* branch,
                               const int* __restrict__ rows, const float* __restrict__ w, int dim,
                               int src_rows, float eps, float offset, int* err) {
    __shared__ float scratch[33];
    extern __shared__ float srow[];  // dim floats
    const int r = blockIdx.x;
    int src = rows ? rows[r] : r;
    if (src < 0 || src >= src_rows) {
        if (threadIdx.x == 0) atomicOr(err, XB_ERR_BAD_ROW);
        src = 0;
    }
    const T* xr = x + (size_t)src * dim;
    const T* br = branch ? branch + (size_t)src * dim : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = to_f32<T>(xr[i]);
        if (br) v = to_f32<T>(from_f32<T>(v + to_f32<T>(br[i])));
        srow[i] = v;
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float inv = rsqrtf(total / (float)dim + eps);
    T* o = out + (size_t)r * dim;
    T* so = sum_out ? sum_out + (size_t)r * dim : nullptr;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = srow[i];
        if (so) so[i] = from_f32<T>(v);
        o[i] = from_f32<T>(v * inv * (offset + w[i]));
    }
}

XB_EXPORT int xb_rmsnorm(int dtype, void* out, void* sum_out, const void* x, const void* branch,
                         const int* rows, const float* w, int nrows, int dim, int src_rows,
                         float eps, float offset, int* err, cudaStream_t stream) {
    if (nrows <= 0) return 0;
    const size_t smem = (size_t)dim * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    const int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128);
    if (dtype == XB_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        rmsnorm_kernel<float><<<nrows, threads, smem, stream>>>((float*)out, (float*)sum_out, (const float*)x, (const float*)branch, rows, w, dim, src_rows, eps, offset, err);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(rmsnorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        rmsnorm_kernel<__nv_bfloat16><<<nrows, threads, smem, stream>>>((__nv_bfloat16*)out, (__nv_bfloat16*)sum_out, (const __nv_bfloat16*)x, (const __nv_bfloat16*)branch, rows, w, dim, src_rows, eps, offset, err);
    }
    return xb_launch_status();
}

// ------------------------------------------------------------------------------------------
// out[t] = x[t] + branch[t]  (float32 sum, rounded to T); used where no norm follows.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void add_kernel(T* out, const T* x, const T* branch, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_f32<T>(to_f32<T>(x[i]) + to_f32<T>(branch[i]));
}

XB_EXPORT int xb_add(int dtype, void* out, const void* x, const void* branch, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int threads = 256;
    const unsigned blocks = (unsigned)((n + threads - 1) / threads);
    if (dtype == XB_F32)
        add_kernel<float><<<blocks, threads, 0, stream>>>((float*)out, (const float*)x, (const float*)branch, (size_t)n);
    else
        add_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)x, (const __nv_bfloat16*)branch, (size_t)n);
    return xb_launch_status();
}

// ------------------------------------------------------------------------------------------
// Plain matrix product  out[M, N] = a[M, K] . w[N, K]^T  with float32 FMA accumulation.
// 64x64 tile, 16-deep panels, 256 threads with 4x4 outputs each.  k runs in order for every
// output, so a row's result does not depend on M.
// ------------------------------------------------------------------------------------------
template <typename TA, typename TW, typename TO>
__global__ void gemm_plain_kernel(TO* __restrict__ out, const TA* __restrict__ a,
                                  const TW* __restrict__ w, int M, int N, int K) {
    constexpr int BM = 64, BN = 64, BK = 16;
    __shared__ float sa[BK][BM + 1];
    __shared__ float sw[BK][BN + 1];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int idx = threadIdx.x; idx < BM * BK; idx += 256) {
            const int r = idx / BK, c = idx % BK;
            const int gm = m0 + r, gk = k0 + c;
            sa[c][r] = (gm < M && gk < K) ? to_f32<TA>(a[(size_t)gm * K + gk]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < BN * BK; idx += 256) {
            const int r = idx / BK, c = idx % BK;
            const int gn = n0 + r, gk = k0 + c;
            sw[c][r] = (gn < N && gk < K) ? to_f32<TW>(w[(size_t)gn * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = sw[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) out[(size_t)gm * N + gn] = from_f32<TO>(acc[i][j]);
        }
    }
}

template <typename TA, typename TW, typename TO>
static int gemm_plain_launch(void* out, const void* a, const void* w, int M, int N, int K, cudaStream_t stream) {
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    gemm_plain_kernel<TA, TW, TO><<<grid, 256, 0, stream>>>((TO*)out, (const TA*)a, (const TW*)w, M, N, K);
    return xb_launch_status();
}

// a_dtype / w_dtype / out_dtype are element type codes.
XB_EXPORT int xb_gemm_plain(int a_dtype, int w_dtype, int out_dtype, void* out, const void* a,
                            const void* w, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    typedef __nv_bfloat16 bf;
    const int code = a_dtype * 4 + w_dtype * 2 + out_dtype;
    switch (code) {
        case 0: return gemm_plain_launch<float, float, float>(out, a, w, M, N, K, stream);
        case 1: return gemm_plain_launch<float, float, bf>(out, a, w, M, N, K, stream);
        case 2: return gemm_plain_launch<float, bf, float>(out, a, w, M, N, K, stream);
        case 3: return gemm_plain_launch<float, bf, bf>(out, a, w, M, N, K, stream);
        case 4: return gemm_plain_launch<bf, float, float>(out, a, w, M, N, K, stream);
        case 5: return gemm_plain_launch<bf, float, bf>(out, a, w, M, N, K, stream);
        case 6: return gemm_plain_launch<bf, bf, float>(out, a, w, M, N, K, stream);
        case 7: return gemm_plain_launch<bf, bf, bf>(out, a, w, M, N, K, stream);
    }
    return (int)cudaErrorInvalidValue;
}

// ------------------------------------------------------------------------------------------
// Rotary tables: cos/sin[pos, j] of angle pos * inv_freq[j], all float32.
// ------------------------------------------------------------------------------------------
__global__ void rope_table_kernel(float* cos_t, float* sin_t, const float* inv_freq, int max_pos, int half) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)max_pos * half) return;
    const int pos = (int)(i / half), j = (int)(i % half);
    const float ang = (float)pos * inv_freq[j];
    float s, c;
    sincosf(ang, &s, &c);
    cos_t[i] = c;
    sin_t[i] = s;
}

XB_EXPORT int xb_rope_table(float* cos_t, float* sin_t, const float* inv_freq, int max_pos, int half, cudaStream_t stream) {
    const size_t n = (size_t)max_pos * half;
    if (n == 0) return 0;
    rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(cos_t, sin_t, inv_freq, max_pos, half);
    return xb_launch_status();
}

// ------------------------------------------------------------------------------------------
// Per-head q/k RMSNorm + rotary encoding + cache write, reading the packed projection once.
//   qkv[t] = [q heads | k heads | v heads], each head `d` wide.
//   q_out[t, h]  = rope(norm(q))            k_cache[page, g, off] = rope(norm(k))
//   v_cache[page, g, off] = v               page = table[b, pos / page_size]
// Cache layout: [num_pages, kv_heads, page_size, d].  One warp per (token, head).
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void qk_norm_rope_write_kernel(
    T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
    const T* __restrict__ qkv, const float* __restrict__ q_w, const float* __restrict__ k_w,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t,
    const int* __restrict__ positions, const int* __restrict__ req_of_token,
    const int* __restrict__ block_table, int table_stride, int nh, int nkv, int d, int rot,
    int interleaved, int page_size, int num_pages, int max_pos, float eps, int write_kv, int* err) {
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int pos = positions[t];
    const int total_heads = nh + 2 * nkv;
    const int half = rot / 2;
    const T* row = qkv + (size_t)t * total_heads * d;
    // destination of this token's k/v rows
    long long kv_row = -1;
    if (write_kv && req_of_token[t] >= 0) {  // request -1 marks a padding token
        const int b = req_of_token[t];
        const int page = block_table[(size_t)b * table_stride + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicOr(err, XB_ERR_BAD_PAGE);
        } else {
            kv_row = (long long)page * nkv * page_size + (pos % page_size);  // + g * page_size
        }
    }
    // a position the table does not hold is reported; the row read instead keeps the access in bounds
    if (cos_t && (pos < 0 || pos >= max_pos) && req_of_token[t] >= 0 && threadIdx.x == 0) atomicOr(err, XB_ERR_BAD_POSITION);
    const int tp = pos < max_pos ? (pos < 0 ? 0 : pos) : max_pos - 1;
    for (int h = warp; h < total_heads; h += nwarps) {
        const T* x = row + (size_t)h * d;
        const bool is_q = h < nh, is_k = h >= nh && h < nh + nkv;
        T* dst;
        if (is_q) {
            dst = q_out + ((size_t)t * nh + h) * d;
        } else {
            if (!write_kv || kv_row < 0) continue;
            const int g = is_k ? h - nh : h - nh - nkv;
            dst = (is_k ? k_cache : v_cache) + (size_t)(kv_row + (long long)g * page_size) * d;
        }
        if (!is_q && !is_k) {  // value head: copy
            for (int i = lane; i < d; i += 32) dst[i] = x[i];
            continue;
        }
        const float* nw = is_q ? q_w : k_w;
        float inv = 1.f;
        if (nw) {
            float ss = 0.f;
            for (int i = lane; i < d; i += 32) {
                const float v = to_f32<T>(x[i]);
                ss += v * v;
            }
            ss = warp_sum(ss);
            inv = rsqrtf(ss / (float)d + eps);
        }
        if (cos_t) {
            for (int j = lane; j < half; j += 32) {
                const int i0 = interleaved ? 2 * j : j;
                const int i1 = interleaved ? 2 * j + 1 : j + half;
                float a = to_f32<T>(x[i0]), b = to_f32<T>(x[i1]);
                if (nw) {
                    a = a * inv * nw[i0];
                    b = b * inv * nw[i1];
                }
                const float c = cos_t[(size_t)tp * half + j], s = sin_t[(size_t)tp * half + j];
                dst[i0] = from_f32<T>(a * c - b * s);
                dst[i1] = from_f32<T>(a * s + b * c);
            }
            for (int i = rot + lane; i < d; i += 32) {
                float a = to_f32<T>(x[i]);
                if (nw) a = a * inv * nw[i];
                dst[i] = from_f32<T>(a);
            }
        } else {
            for (int i = lane; i < d; i += 32) {
                float a = to_f32<T>(x[i]);
                if (nw) a = a * inv * nw[i];
                dst[i] = from_f32<T>(a);
            }
        }
    }
}

XB_EXPORT int xb_qk_norm_rope_write(
    int dtype, void* q_out, void* k_cache, void* v_cache, const void* qkv, const float* q_w,
    const float* k_w, const float* cos_t, const float* sin_t, const int* positions,
    const int* req_of_token, const int* block_table, int table_stride, int tokens, int nh, int nkv,
    int d, int rot, int interleaved, int page_size, int num_pages, int max_pos, float eps,
    int write_kv, int* err, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const int threads = 128;
    if (dtype == XB_F32)
        qk_norm_rope_write_kernel<float><<<tokens, threads, 0, stream>>>(
            (float*)q_out, (float*)k_cache, (float*)v_cache, (const float*)qkv, q_w, k_w, cos_t, sin_t,
            positions, req_of_token, block_table, table_stride, nh, nkv, d, rot, interleaved, page_size,
            num_pages, max_pos, eps, write_kv, err);
    else
        qk_norm_rope_write_kernel<__nv_bfloat16><<<tokens, threads, 0, stream>>>(
            (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, (const __nv_bfloat16*)qkv,
            q_w, k_w, cos_t, sin_t, positions, req_of_token, block_table, table_stride, nh, nkv, d, rot,
            interleaved, page_size, num_pages, max_pos, eps, write_kv, err);
    return xb_launch_status();
}

// ------------------------------------------------------------------------------------------
// Plain attention over the paged cache.  One warp per (token, head); keys are visited in
// position order with a running maximum, so a query's result depends only on its own position
// and the keys before it.  Scores, softmax and the value sum are float32.
//   keys seen by a query at position p:  max(0, p - window + 1) .. p   (window <= 0: from 0)
// ------------------------------------------------------------------------------------------
template <typename T, int MAXE>
__global__ void attention_plain_kernel(
    T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ k_cache,
    const T* __restrict__ v_cache, const int* __restrict__ positions,
    const int* __restrict__ req_of_token, const int* __restrict__ block_table, int table_stride,
    int nh, int nkv, int d, int page_size, int num_pages, int window, float scale, int* err) {
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31;
    const int h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (h >= nh) return;
    const int g = h / (nh / nkv);
    const int pos = positions[t];
    const int b = req_of_token[t];
    if (b < 0) {  // padding token
        T* o = out + ((size_t)t * nh + h) * d;
        for (int i = lane; i < d; i += 32) o[i] = from_f32<T>(0.f);
        return;
    }
    const int* table = block_table + (size_t)b * table_stride;
    const T* qv = q + ((size_t)t * nh + h) * d;
    float qr[MAXE], acc[MAXE];
#pragma unroll
    for (int e = 0; e < MAXE; ++e) {
        const int i = e * 32 + lane;
        qr[e] = i < d ? to_f32<T>(qv[i]) * scale : 0.f;
        acc[e] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    for (int j = lo; j <= pos; ++j) {
        const int page = table[j / page_size];
        if (page < 0 || page >= num_pages) {
            if (lane == 0) atomicOr(err, XB_ERR_BAD_PAGE);
            continue;
        }
        const size_t rowi = ((size_t)page * nkv + g) * page_size + (j % page_size);
        const T* kr = k_cache + rowi * d;
        const T* vr = v_cache + rowi * d;
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < MAXE; ++e) {
            const int i = e * 32 + lane;
            if (i < d) s = fmaf(qr[e], to_f32<T>(kr[i]), s);
        }
        s = warp_sum(s);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);  // exp(-inf) = 0 on the first key
        const float p = expf(s - m_new);
        l = l * corr + p;
#pragma unroll
        for (int e = 0; e < MAXE; ++e) {
            const int i = e * 32 + lane;
            if (i < d) acc[e] = acc[e] * corr + p * to_f32<T>(vr[i]);
        }
        m = m_new;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    T* o = out + ((size_t)t * nh + h) * d;
#pragma unroll
    for (int e = 0; e < MAXE; ++e) {
        const int i = e * 32 + lane;
        if (i < d) o[i] = from_f32<T>(acc[e] * inv);
    }
}

template <typename T>
static int attention_plain_launch(void* out, const void* q, const void* kc, const void* vc,
                                  const int* positions, const int* req_of_token, const int* block_table,
                                  int table_stride, int tokens, int nh, int nkv, int d, int page_size,
                                  int num_pages, int window, float scale, int* err, cudaStream_t stream) {
    dim3 grid(tokens, (nh + 3) / 4);
#define XB_ATT(MAXE)                                                                              \
    attention_plain_kernel<T, MAXE><<<grid, 128, 0, stream>>>(                                    \
        (T*)out, (const T*)q, (const T*)kc, (const T*)vc, positions, req_of_token, block_table,   \
        table_stride, nh, nkv, d, page_size, num_pages, window, scale, err)
    if (d <= 64) XB_ATT(2);
    else if (d <= 128) XB_ATT(4);
    else if (d <= 256) XB_ATT(8);
    else if (d <= 512) XB_ATT(16);
    else return (int)cudaErrorInvalidValue;
#undef XB_ATT
    return xb_launch_status();
}

XB_EXPORT int xb_attention_plain(int dtype, void* out, const void* q, const void* k_cache,
                                 const void* v_cache, const int* positions, const int* req_of_token,
                                 const int* block_table, int table_stride, int tokens, int nh, int nkv,
                                 int d, int page_size, int num_pages, int window, float scale, int* err,
                                 cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (dtype == XB_F32)
        return attention_plain_launch<float>(out, q, k_cache, v_cache, positions, req_of_token, block_table,
                                             table_stride, tokens, nh, nkv, d, page_size, num_pages, window, scale, err, stream);
    return attention_plain_launch<__nv_bfloat16>(out, q, k_cache, v_cache, positions, req_of_token, block_table,
                                                 table_stride, tokens, nh, nkv, d, page_size, num_pages, window, scale, err, stream);
}

// ------------------------------------------------------------------------------------------
// Gated activation: out[t, i] = silu(gu[t, i]) * gu[t, I + i], silu(z) = z / (1 + exp(-z)).
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(T* __restrict__ out, const T* __restrict__ gu, int inter, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t t = i / inter, c = i % inter;
    const float g = to_f32<T>(gu[t * 2 * inter + c]);
    const float u = to_f32<T>(gu[t * 2 * inter + inter + c]);
    out[i] = from_f32<T>(sizeof(T) == 2 ? silu_mul_bf16(g, u) : g / (1.f + expf(-g)) * u);
}

XB_EXPORT int xb_swiglu(int dtype, void* out, const void* gu, int tokens, int inter, cudaStream_t stream) {
    const size_t n = (size_t)tokens * inter;
    if (n == 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == XB_F32)
        swiglu_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, (const float*)gu, inter, n);
    else
        swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)gu, inter, n);
    return xb_launch_status();
}

// ------------------------------------------------------------------------------------------
// Widening copy bf16 -> f32 (logits of the bfloat16 head).
// ------------------------------------------------------------------------------------------
__global__ void widen_kernel(float* out, const __nv_bfloat16* in, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __bfloat162float(in[i]);
}
// eight elements per thread with 16-byte accesses (n a multiple of 8, both pointers 16-byte aligned)
__global__ void widen8_kernel(float4* __restrict__ out, const uint4* __restrict__ in, size_t nvec) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nvec) return;
    const uint4 p = in[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&p);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]), c = __bfloat1622float2(h[2]), d = __bfloat1622float2(h[3]);
    out[2 * i] = make_float4(a.x, a.y, b.x, b.y);
    out[2 * i + 1] = make_float4(c.x, c.y, d.x, d.y);
}

XB_EXPORT int xb_widen_bf16(float* out, const void* in, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (n % 8 == 0 && !(((uintptr_t)out | (uintptr_t)in) & 15)) {
        const size_t nvec = (size_t)n / 8;
        widen8_kernel<<<(unsigned)((nvec + 255) / 256), 256, 0, stream>>>((float4*)out, (const uint4*)in, nvec);
        return xb_launch_status();
    }
    widen_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(out, (const __nv_bfloat16*)in, (size_t)n);
    return xb_launch_status();
}
