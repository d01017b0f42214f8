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

// order-preserving map float -> uint32 (larger float, larger key); NaN sorts lowest; the two zeros get one
// key (-0 + 0 is +0), as they compare equal everywhere else
__device__ __forceinline__ uint32_t float_key(float v) {
    if (v != v) return 0u;
    const uint32_t b = __float_as_uint(v + 0.f);
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

// Four Gumbel values of the tokens 4g .. 4g+3 from one Philox block.
__device__ __forceinline__ void gumbel4_of(uint32_t seed_lo, uint32_t seed_hi, uint32_t draw, int g, float out[4]) {
    uint32_t r[4];
    philox4x32_10((uint32_t)g, draw, 0x58494e46u, 0u, seed_lo, seed_hi, r);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float u = ((float)(r[e] >> 9) + 0.5f) * (1.0f / 8388608.0f);
        out[e] = -logf(-logf(u));
    }
}

__device__ __forceinline__ unsigned long long key_of(float v, int i) {
    return ((unsigned long long)float_key(v) << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)i);
}

#define XB_SAMPLE_CHUNK_SMEM 6144   // values of a chunk that are kept in shared memory
#define XB_SAMPLE_POOL 1024         // keys above a chunk's first threshold that are kept in shared memory
#define XB_SAMPLE_CHUNKS_MAX 64

// The `need`-th largest of the n unique 64-bit keys key_at(0) .. key_at(n - 1), or a lower bound of it
// above the next smaller key: `key >= result` holds for exactly the `need` largest (need <= n).  A radix
// select from the top byte down; the whole block takes part (blockDim.x a multiple of 32).  The
// passes end as soon as a bin is needed whole, which for float keys with an index below them is after
// the float's bytes at the latest in practice.
struct SelectShared {
    unsigned int hist[256];
    unsigned long long prefix;
    int need, done;
};
template <typename KeyAt>
__device__ __forceinline__ unsigned long long select_kth(int n, int need, KeyAt key_at, SelectShared& sh) {
    const int tid = threadIdx.x, lane = tid & 31;
    if (tid == 0) {
        sh.prefix = 0ull;
        sh.need = need;
        sh.done = 0;
    }
    __syncthreads();
    for (int pass = 7; pass >= 0; --pass) {
        if (tid < 256) sh.hist[tid] = 0u;
        __syncthreads();
        const unsigned long long prefix = sh.prefix;
        const int shift = pass * 8;
        for (int base = 0; base < n; base += blockDim.x) {   // the same trips for every thread: the match below is warp-wide
            const int i = base + tid;
            unsigned int bin = 256u + (unsigned)lane;        // matches no other lane
            if (i < n) {
                const unsigned long long key = key_at(i);
                if (pass == 7 || (key >> (shift + 8)) == (prefix >> (shift + 8))) bin = (unsigned)(key >> shift) & 255u;
            }
            // the lanes that share the first lane's bin add as one; the others each for themselves
            const unsigned int first = __shfl_sync(0xffffffffu, bin, 0);
            const unsigned int same = __ballot_sync(0xffffffffu, bin == first);
            if (bin == first) {
                if (lane == 0 && bin < 256u) atomicAdd(&sh.hist[bin], (unsigned)__popc(same));
            } else if (bin < 256u) {
                atomicAdd(&sh.hist[bin], 1u);
            }
        }
        __syncthreads();
        if (tid < 32) {
            // the bin in which the count, summed from the top bin down, reaches what is still needed:
            // lane l holds bins 255 - 8l down to 248 - 8l
            unsigned int c[8], sum = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                c[j] = sh.hist[255 - (8 * lane + j)];
                sum += c[j];
            }
            unsigned int incl = sum;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned int t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            const unsigned int want = (unsigned int)sh.need, excl = incl - sum;
            const bool here = excl < want && (incl >= want || lane == 31);
            __syncwarp();
            if (here) {
                unsigned int rem = want - excl;
                int bin = 0;
                bool whole = false;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int b = 255 - (8 * lane + j);
                    if (c[j] >= rem || b == 0) {
                        bin = b;
                        whole = c[j] == rem;   // every key of this bin is wanted: the bytes below decide nothing
                        break;
                    }
                    rem -= c[j];
                }
                sh.need = (int)rem;
                sh.prefix = prefix | ((unsigned long long)bin << shift);
                sh.done = whole ? 1 : 0;
            }
        }
        __syncthreads();
        if (sh.done) break;
    }
    return sh.prefix;
}

#define XB_SAMPLE_FEW 64   // up to this many wanted keys are found through the maxima of groups of four threads

// A threshold that at least n of the block's keys reach (one key per thread, 0: none), found without
// counting them all: the n-th largest of the maxima of the 256 groups of four adjacent threads (each is
// one of the keys, so n keys are >= it; and a group's maximum is a rare value, so not many more are).
// 0 when fewer than n groups hold a key: then every key is wanted.  blockDim.x must be 1024.
__device__ __forceinline__ unsigned long long group_threshold(unsigned long long mine, int n, unsigned long long* gmax /* [256] */,
                                                              unsigned long long* s_t) {
    unsigned long long g = mine, o;
    o = __shfl_xor_sync(0xffffffffu, g, 1);
    g = o > g ? o : g;
    o = __shfl_xor_sync(0xffffffffu, g, 2);
    g = o > g ? o : g;
    __syncthreads();   // whoever read gmax or s_t before is done
    if ((threadIdx.x & 3) == 0) gmax[threadIdx.x >> 2] = g;
    if (threadIdx.x == 0) *s_t = 0ull;
    __syncthreads();
    if (threadIdx.x < 256) {
        const unsigned long long me = gmax[threadIdx.x];
        int larger = 0;
#pragma unroll 8
        for (int j = 0; j < 256; ++j) larger += gmax[j] > me ? 1 : 0;
        if (me != 0ull && larger == n - 1) *s_t = me;   // keys are unique: one group at most
    }
    __syncthreads();
    return *s_t;
}

// The `n` largest of pool[0 .. m), in descending order, to dst[0 .. n): every key is placed by the number of
// keys above it (m is small: a few times n).  Keys are unique.
__device__ __forceinline__ void place_largest(const unsigned long long* pool, int m, int n, unsigned long long* dst, bool write) {
    for (int i = threadIdx.x; i < m; i += blockDim.x) {
        const unsigned long long me = pool[i];
        int larger = 0;
        for (int j = 0; j < m; ++j) larger += pool[j] > me ? 1 : 0;
        if (write && larger < n) dst[larger] = me;
    }
}

// Scratch of the sampler, per row: a candidate counter and a ticket (both zero between launches),
// candidate keys, partial results of the chunks.  The arrays are laid out for the buffer's capacity
// (the most rows it will ever see), not for a launch's rows: the counters of a smaller batch must
// not fall where a larger batch left keys.
struct SampleScratch {
    int* count;                 // [capacity]
    int* ticket;                // [capacity]
    unsigned long long* cand;   // [capacity][XB_TOPK_MAX]
    Best* part;                 // [capacity][XB_SAMPLE_CHUNKS_MAX]
};

// Grid (chunks, rows): a row's vocabulary is cut into chunks of whole Philox blocks (4 tokens); every
// CTA reduces its chunk - to its best token, or to its k largest - and the CTA that finishes last
// among a row's chunks (a ticket) makes the draw from those partial results.  Rows with a top-k use
// at most 1024 / k chunks, so that the candidates of all chunks fit the final sort.
__global__ void __launch_bounds__(1024)
sample_kernel(int* __restrict__ out_tokens, const float* __restrict__ logits, const SampleParams* __restrict__ params,
              int vocab, int grid_chunks, SampleScratch sc, int* __restrict__ err_word) {
    // the step's error word travels to the host behind the tokens, in the same copy (what this launch
    // itself reports reaches the host with the next one)
    if (err_word != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) out_tokens[gridDim.y] = *err_word;
    __shared__ Best sbest[32];
    __shared__ SelectShared sel;
    __shared__ unsigned long long cand_key[XB_TOPK_MAX];
    __shared__ float cand_p[XB_TOPK_MAX];
    __shared__ __align__(8) float s_vals[XB_SAMPLE_CHUNK_SMEM];
    __shared__ unsigned long long pool[XB_SAMPLE_POOL];
    __shared__ unsigned long long gmax[256];
    __shared__ unsigned long long s_t;
    __shared__ int s_need, s_base, s_keep, s_last;

    const int r = blockIdx.y;
    const SampleParams p = params[r];
    const float* row = logits + (size_t)r * vocab;
    const bool greedy = !(p.temperature >= 1e-7f);
    const bool use_p = p.top_p > 0.f && p.top_p < 1.f;
    const bool truncated = !greedy && (p.top_k > 0 || use_p);
    const float inv_t = greedy ? 1.f : 1.f / p.temperature;
    int k = p.top_k > 0 ? p.top_k : 256;  // top-p alone looks at the 256 largest, as the reference's device sampler does
    if (k > XB_TOPK_MAX) k = XB_TOPK_MAX;
    if (k > vocab) k = vocab;

    // this row's chunks
    int chunks = truncated ? min(grid_chunks, XB_TOPK_MAX / k) : grid_chunks;
    if (chunks < 1) chunks = 1;
    const int chunk_n = ((vocab + chunks - 1) / chunks + 3) & ~3;
    chunks = (vocab + chunk_n - 1) / chunk_n;
    if ((int)blockIdx.x >= chunks) return;
    const int lo = (int)blockIdx.x * chunk_n, hi = min(vocab, lo + chunk_n);

    if (!truncated) {
        Best b{0.f, -1};
        for (int g4 = (lo >> 2) + (int)threadIdx.x; g4 * 4 < hi; g4 += blockDim.x) {
            float noise[4] = {0.f, 0.f, 0.f, 0.f};
            if (!greedy) gumbel4_of(p.seed_lo, p.seed_hi, p.draw, g4, noise);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = g4 * 4 + e;
                if (i < hi) {
                    float v = row[i];
                    if (!greedy) v = v * inv_t + noise[e];
                    b = better(b, Best{v, i});
                }
            }
        }
        b = block_best(b, sbest);
        if (threadIdx.x == 0) sc.part[(size_t)r * XB_SAMPLE_CHUNKS_MAX + blockIdx.x] = b;
    } else {
        // ---- the chunk's k largest by (value, then lower index) --------------------------------------------
        // Few wanted among many: every thread keeps the largest key of the elements it reads; the kc-th
        // largest of those 1024 maxima is a threshold T that at least kc elements reach, so the chunk's kc
        // largest are among the elements >= T - about kc of them, since a thread's maximum is a rare value.
        // They are gathered in shared memory and the kc-th is selected among them.  The chunk is read
        // twice and counted once.  Otherwise (many wanted, or more than the pool holds reached T): a radix
        // select over the whole chunk.
        const int n_chunk = hi - lo;
        const bool cached = n_chunk <= XB_SAMPLE_CHUNK_SMEM;
        const int kc = min(k, n_chunk);
        unsigned long long mine = 0ull;   // below every key: a key's low half is 2^32 - 1 - index > 0
        for (int i = threadIdx.x; i < n_chunk; i += blockDim.x) {
            const float v = row[lo + i];
            if (cached) s_vals[i] = v;
            const unsigned long long key = key_of(v, lo + i);
            mine = key > mine ? key : mine;
        }
        auto key_at = [&](int i) { return key_of(cached ? s_vals[i] : row[lo + i], lo + i); };
        const int holders = min(n_chunk, (int)blockDim.x);   // threads that read an element
        bool gathered = kc <= XB_SAMPLE_POOL / 4 && holders >= 4 * kc;
        const bool few = gathered && kc <= XB_SAMPLE_FEW;
        unsigned long long kth = 0ull;
        int pooled = 0;
        if (gathered) {
            unsigned long long T;
            if (few) {
                T = group_threshold(mine, kc, gmax, &s_t);
                if (T == 0ull) T = 1ull;    // fewer groups than wanted keys hold any: every element (keys are >= 1)
            } else {
                cand_key[threadIdx.x] = mine;   // (free until the row's last CTA needs it)
                T = select_kth(holders, kc, [&](int i) { return cand_key[i]; }, sel);
            }
            if (threadIdx.x == 0) s_need = 0;
            __syncthreads();
            for (int i = threadIdx.x; i < n_chunk; i += blockDim.x) {
                const unsigned long long key = key_at(i);
                if (key >= T) {
                    const int at = atomicAdd(&s_need, 1);
                    if (at < XB_SAMPLE_POOL) pool[at] = key;
                }
            }
            __syncthreads();
            pooled = s_need;
            gathered = pooled <= XB_SAMPLE_POOL;
            if (gathered && !few) kth = pooled > kc ? select_kth(pooled, kc, [&](int i) { return pool[i]; }, sel) : T;
        }
        if (!gathered) kth = select_kth(n_chunk, kc, key_at, sel);   // keys of the chunk's kc largest are >= kth; keys are unique
        __syncthreads();
        if (threadIdx.x == 0) s_base = atomicAdd(&sc.count[r], kc);   // room for this chunk's candidates
        __syncthreads();
        // a counter that was not zero at launch (scratch shared with something else) must not turn
        // into a write outside the row's candidates: report it and write nothing
        const bool room = s_base >= 0 && s_base + kc <= XB_TOPK_MAX;
        if (!room && threadIdx.x == 0 && err_word != nullptr) atomicOr(err_word, XB_ERR_SCRATCH);
        unsigned long long* dst = sc.cand + (size_t)r * XB_TOPK_MAX + (room ? s_base : 0);
        if (threadIdx.x == 0) s_need = 0;
        __syncthreads();
        if (gathered && few) {
            place_largest(pool, pooled, kc, dst, room);
        } else {
            const int from = gathered ? pooled : n_chunk;
            for (int i = threadIdx.x; i < from; i += blockDim.x) {
                const unsigned long long key = gathered ? pool[i] : key_at(i);
                if (key >= kth) {
                    const int at = atomicAdd(&s_need, 1);
                    if (room && at < kc) dst[at] = key;
                }
            }
        }
    }
    // ---- the CTA that finishes last among the row's chunks makes the draw ---------------------------------
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int mine = atomicAdd(&sc.ticket[r], 1);
        s_last = mine == chunks - 1;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (!truncated) {
        Best b{0.f, -1};
        if ((int)threadIdx.x < chunks) {
            const Best* src = sc.part + (size_t)r * XB_SAMPLE_CHUNKS_MAX + threadIdx.x;
            b.v = __ldcg(&src->v);
            b.i = __ldcg(&src->i);
        }
        b = block_best(b, sbest);
        if (threadIdx.x == 0) {
            out_tokens[r] = b.i;
            sc.ticket[r] = 0;
        }
        return;
    }
    const int total = max(0, min(__ldcg(&sc.count[r]), XB_TOPK_MAX));
    for (int i = threadIdx.x; i < XB_TOPK_MAX; i += blockDim.x)
        cand_key[i] = i < total ? __ldcg(sc.cand + (size_t)r * XB_TOPK_MAX + i) : 0ull;
    __syncthreads();
    if (threadIdx.x == 0) {   // ready for the next launch
        sc.ticket[r] = 0;
        sc.count[r] = 0;
    }
    const int n = total < k ? total : k;
    if (n <= XB_SAMPLE_FEW && total > n) {
        // few wanted: a threshold from the groups' maxima, the candidates that reach it gathered and placed in order
        const unsigned long long my_key = (int)threadIdx.x < total ? cand_key[threadIdx.x] : 0ull;
        unsigned long long T = group_threshold(my_key, n, gmax, &s_t);
        if (T == 0ull) T = 1ull;
        if (threadIdx.x == 0) s_need = 0;
        __syncthreads();
        if (my_key >= T) pool[atomicAdd(&s_need, 1)] = my_key;   // at most `total` <= 1024 of them
        __syncthreads();
        const int m = s_need;
        for (int i = threadIdx.x; i < XB_TOPK_MAX; i += blockDim.x) cand_key[i] = 0ull;
        __syncthreads();
        place_largest(pool, m, n, cand_key, true);
        __syncthreads();
    } else {
    // the row's n largest among the chunks' candidates (a select, as above), moved to the front ...
    if (total > n) {
        unsigned long long* top = reinterpret_cast<unsigned long long*>(s_vals);   // the chunk's values are done with
        const unsigned long long kth = select_kth(total, n, [&](int i) { return cand_key[i]; }, sel);
        if (threadIdx.x == 0) s_need = 0;
        __syncthreads();
        for (int i = threadIdx.x; i < total; i += blockDim.x) {
            const unsigned long long key = cand_key[i];
            if (key >= kth) {
                const int at = atomicAdd(&s_need, 1);
                if (at < n) top[at] = key;
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < XB_TOPK_MAX; i += blockDim.x) cand_key[i] = i < n ? top[i] : 0ull;
        __syncthreads();
    }
    // ... and put in descending order: a bitonic sort over the next power of two
    int sort_n = 2;
    while (sort_n < n) sort_n <<= 1;
    for (int size = 2; size <= sort_n; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            const int i = threadIdx.x;
            const int j = i ^ stride;
            if (i < sort_n && j > i) {
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
            float total_p = 0.f;
            for (int i = 0; i < n; ++i) total_p += cand_p[i];
            float cum = 0.f;
            keep = 0;
            for (int i = 0; i < n; ++i) {
                if (cum >= p.top_p) break;
                cum += cand_p[i] / total_p;
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

// Bytes of scratch for a sampler that sees at most `capacity` rows in a launch (zero before the first
// launch; the kernel leaves it zero where it must be).
XB_EXPORT long long xb_sample_scratch_bytes(int capacity) {
    return (long long)capacity * (8 + XB_TOPK_MAX * 8 + XB_SAMPLE_CHUNKS_MAX * (long long)sizeof(Best));
}

// `err_word` (nullable): a device int that is copied to out_tokens[rows].  `scratch`: at least
// xb_sample_scratch_bytes(capacity) bytes, 8-byte aligned, laid out by `capacity` (the same value in
// every call that shares the buffer), rows <= capacity.
XB_EXPORT int xb_sample(int* out_tokens, float* logits, const void* params, const int* history,
                        int rows, int capacity, int vocab, int apply_penalties, void* scratch, int* err_word,
                        cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (!scratch || ((uintptr_t)scratch & 7) || rows > capacity) return (int)cudaErrorInvalidValue;
    if (apply_penalties) penalties_kernel<<<rows, 128, 0, stream>>>(logits, (const SampleParams*)params, history, vocab);
    SampleScratch sc;
    unsigned char* base = (unsigned char*)scratch;
    sc.count = (int*)base;
    sc.ticket = sc.count + capacity;
    base += (size_t)capacity * 8;
    sc.cand = (unsigned long long*)base;
    base += (size_t)capacity * XB_TOPK_MAX * 8;
    sc.part = (Best*)base;
    int chunks = 148 / rows;   // one CTA of 1024 threads per SM of a 148-SM part (its registers fill the SM): one wave
    if (chunks < 1) chunks = 1;
    if (chunks > XB_SAMPLE_CHUNKS_MAX) chunks = XB_SAMPLE_CHUNKS_MAX;
    sample_kernel<<<dim3(chunks, rows), 1024, 0, stream>>>(out_tokens, logits, (const SampleParams*)params, vocab, chunks, sc, err_word);
    return xb_launch_status();
}

XB_EXPORT int xb_sample_params_size() { return (int)sizeof(SampleParams); }
