// Token sampling on the device: greedy, temperature, top-k, top-p, top-k-then-top-p, and the
// frequency / presence penalties.
//
// A draw from softmax(logits / T) restricted to a kept set is made as
//     argmax over the kept set of  logits[i] / T + G(seed, n, i),   G = -log(-log(u)),
// with u a uniform from Philox4x32-10 keyed by the request's seed, counter (i / 4, n, ...), n the
// number of tokens the request has drawn so far.  The noise of a token depends only on
// (seed, n, i): what else is in the batch cannot change a request's samples.
#include "common.cuh"

#define XB_TOPK_MAX 1024

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                              uint32_t k0, uint32_t k1, uint32_t out[4]) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

__device__ __forceinline__ float gumbel_of(uint32_t seed_lo, uint32_t seed_hi, uint32_t draw, int i) {
    uint32_t r[4];
    philox4x32_10((uint32_t)i >> 2, draw, 0x58494e46u, 0u, seed_lo, seed_hi, r);
    const uint32_t w = r[i & 3];
    const float u = ((float)(w >> 9) + 0.5f) * (1.0f / 8388608.0f);  // in (0, 1), exact in float32
    return -logf(-logf(u));
}

// order-preserving map float -> uint32 (larger float, larger key); NaN sorts lowest
__device__ __forceinline__ uint32_t float_key(float v) {
    if (v != v) return 0u;
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct Best {
    float v;
    int i;
};
__device__ __forceinline__ Best better(Best a, Best b) {
    if (b.i < 0) return a;
    if (a.i < 0) return b;
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}
__device__ __forceinline__ Best block_best(Best x, Best* scratch /* 32 */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best y;
        y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
        x = better(x, y);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = x;
    __syncthreads();
    if (warp == 0) {
        Best y = lane < nwarps ? scratch[lane] : Best{0.f, -1};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best z;
            z.v = __shfl_xor_sync(0xffffffffu, y.v, o);
            z.i = __shfl_xor_sync(0xffffffffu, y.i, o);
            y = better(y, z);
        }
        if (lane == 0) scratch[0] = y;
    }
    __syncthreads();
    return scratch[0];
}

// Per-row parameters, one struct per logits row.
struct SampleParams {
    float temperature;   // < 1e-7: greedy
    int top_k;           // <= 0: off
    float top_p;         // outside (0, 1): off
    uint32_t seed_lo, seed_hi;
    uint32_t draw;       // how many tokens this request has drawn before
    float frequency_penalty, presence_penalty;
    int history_offset;  // into the history array
    int history_len;     // tokens the penalties count (0: none)
};

// logits[tok] -= count * frequency + (count > 0) * presence over the row's history.
__global__ void penalties_kernel(float* logits, const SampleParams* params, const int* history, int vocab) {
    const int r = blockIdx.x;
    const SampleParams p = params[r];
    if (p.history_len <= 0 || (p.frequency_penalty == 0.f && p.presence_penalty == 0.f)) return;
    const int* h = history + p.history_offset;
    float* row = logits + (size_t)r * vocab;
    for (int i = threadIdx.x; i < p.history_len; i += blockDim.x) {
        const int tok = h[i];
        if (tok < 0 || tok >= vocab) continue;
        int count = 0;
        bool first = true;
        for (int j = 0; j < p.history_len; ++j) {
            if (h[j] == tok) {
                ++count;
                if (j < i) first = false;
            }
        }
        if (first) row[tok] = row[tok] - (float)count * p.frequency_penalty - p.presence_penalty;
    }
}

__global__ void __launch_bounds__(1024)
sample_kernel(int* __restrict__ out_tokens, const float* __restrict__ logits,
              const SampleParams* __restrict__ params, int vocab) {
    __shared__ Best sbest[32];
    __shared__ unsigned int hist[256];
    __shared__ unsigned long long cand_key[XB_TOPK_MAX];
    __shared__ float cand_p[XB_TOPK_MAX];
    __shared__ unsigned long long s_prefix;
    __shared__ int s_need, s_count, s_keep;

    const int r = blockIdx.x;
    const SampleParams p = params[r];
    const float* row = logits + (size_t)r * vocab;
    const bool greedy = !(p.temperature >= 1e-7f);
    const bool use_p = p.top_p > 0.f && p.top_p < 1.f;
    const bool truncated = !greedy && (p.top_k > 0 || use_p);
    const float inv_t = greedy ? 1.f : 1.f / p.temperature;

    if (!truncated) {
        Best b{0.f, -1};
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            float v = row[i];
            if (!greedy) v = v * inv_t + gumbel_of(p.seed_lo, p.seed_hi, p.draw, i);
            b = better(b, Best{v, i});
        }
        b = block_best(b, sbest);
        if (threadIdx.x == 0) out_tokens[r] = b.i;
        return;
    }

    // ---- the k largest by (value, then lower index): radix select on 64-bit keys ------------
    int k = p.top_k > 0 ? p.top_k : 256;  // top-p alone looks at the 256 largest, as the reference's device sampler does
    if (k > XB_TOPK_MAX) k = XB_TOPK_MAX;
    if (k > vocab) k = vocab;
    if (threadIdx.x == 0) {
        s_prefix = 0ull;
        s_need = k;
    }
    __syncthreads();
    for (int pass = 7; pass >= 0; --pass) {
        if (threadIdx.x < 256) hist[threadIdx.x] = 0u;
        __syncthreads();
        const unsigned long long prefix = s_prefix;
        const int shift = pass * 8;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const unsigned long long key = ((unsigned long long)float_key(row[i]) << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)i);
            if (pass == 7 || (key >> (shift + 8)) == (prefix >> (shift + 8)))
                atomicAdd(&hist[(unsigned)(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int need = s_need;
            int bin = 255;
            for (; bin > 0; --bin) {
                if ((int)hist[bin] >= need) break;
                need -= (int)hist[bin];
            }
            s_need = need;
            s_prefix = prefix | ((unsigned long long)bin << shift);
        }
        __syncthreads();
    }
    const unsigned long long kth = s_prefix;  // the k-th largest key; keys are unique
    if (threadIdx.x == 0) s_count = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const unsigned long long key = ((unsigned long long)float_key(row[i]) << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)i);
        if (key >= kth) {
            const int at = atomicAdd(&s_count, 1);
            if (at < XB_TOPK_MAX) cand_key[at] = key;
        }
    }
    __syncthreads();
    const int n = s_count < k ? s_count : k;
    for (int i = n + threadIdx.x; i < XB_TOPK_MAX; i += blockDim.x) cand_key[i] = 0ull;
    __syncthreads();
    // bitonic sort, descending
    for (int size = 2; size <= XB_TOPK_MAX; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            const int i = threadIdx.x;
            const int j = i ^ stride;
            if (j > i) {
                const bool desc = (i & size) == 0;
                const unsigned long long a = cand_key[i], b = cand_key[j];
                if (desc ? (a < b) : (a > b)) {
                    cand_key[i] = b;
                    cand_key[j] = a;
                }
            }
            __syncthreads();
        }
    }
    // ---- probabilities of the candidates, renormalised; nucleus cut ---------------------------
    {
        const int i = threadIdx.x;
        if (i < n) {
            const int idx0 = (int)(0xFFFFFFFFu - (uint32_t)(cand_key[0] & 0xFFFFFFFFull));
            const int idx = (int)(0xFFFFFFFFu - (uint32_t)(cand_key[i] & 0xFFFFFFFFull));
            cand_p[i] = expf((row[idx] - row[idx0]) * inv_t);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int keep = n;
        if (use_p) {
            float total = 0.f;
            for (int i = 0; i < n; ++i) total += cand_p[i];
            float cum = 0.f;
            keep = 0;
            for (int i = 0; i < n; ++i) {
                if (cum >= p.top_p) break;
                cum += cand_p[i] / total;
                ++keep;
            }
        }
        s_keep = keep;
    }
    __syncthreads();
    Best b{0.f, -1};
    if ((int)threadIdx.x < s_keep) {
        const int idx = (int)(0xFFFFFFFFu - (uint32_t)(cand_key[threadIdx.x] & 0xFFFFFFFFull));
        b = Best{row[idx] * inv_t + gumbel_of(p.seed_lo, p.seed_hi, p.draw, idx), idx};
    }
    b = block_best(b, sbest);
    if (threadIdx.x == 0) out_tokens[r] = b.i;
}

XB_EXPORT int xb_sample(int* out_tokens, float* logits, const void* params, const int* history,
                        int rows, int vocab, int apply_penalties, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (apply_penalties) penalties_kernel<<<rows, 128, 0, stream>>>(logits, (const SampleParams*)params, history, vocab);
    sample_kernel<<<rows, 1024, 0, stream>>>(out_tokens, logits, (const SampleParams*)params, vocab);
    return xb_launch_status();
}

XB_EXPORT int xb_sample_params_size() { return (int)sizeof(SampleParams); }
