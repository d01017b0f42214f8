// Per-head q/k RMSNorm + rotary encoding + cache write for one (token, head), shared by the
// stand-alone bfloat16 kernel and by the q/k/v matrix product that finishes its tile this way.
// Both callers feed it the same bfloat16-rounded projection values and run the same arithmetic in
// the same order, so their results are identical bit for bit.
//
// A group of LPH lanes owns one (token, head); lane i of the group holds the 8-element vectors
// i and i + d/16 of the head (the two halves that a NeoX rotation pairs), so d = 16 * LPH' with
// LPH' <= LPH lanes active.  The interleaved layout pairs elements inside a vector instead.
#pragma once
#include "common.cuh"

namespace xbqk {

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

// Everything but the projection values themselves.
struct QkArgs {
    __nv_bfloat16* q_out;          // [tokens, nh, d]
    __nv_bfloat16* k_cache;        // [pages, nkv, page_size, d]
    __nv_bfloat16* v_cache;
    const float* q_w;              // [d] or null: no norm
    const float* k_w;
    const float* cos_t;            // [max_pos, rot / 2] or null: no rotation
    const float* sin_t;
    const int* positions;          // [tokens]
    const int* req_of_token;       // [tokens]; < 0: padding, nothing is cached
    const int* block_table;        // [requests, table_stride]
    int table_stride, nh, nkv, d, rot, interleaved, page_size, num_pages, max_pos;
    float eps;
    int write_kv;
};

// What a lane needs beside the values: fetched from what the host sent before the step's first
// kernel (positions, block tables) and from constants (norm weights, rotation tables), so a caller
// may run `qk_prepare` while the producer of the values is still at work.
struct QkItem {
    __nv_bfloat16* dst;
    const float* cr;
    const float* sr;
    float wa[8], wb[8], rc[8], rs[8];
    bool normed, neox, rotated;
};

__device__ __forceinline__ QkItem qk_prepare(const QkArgs& A, int t, int h, int li, bool live, int* err) {
    QkItem it;
    const int lanes = A.d / 16, half_vecs = A.d / 16;
    const bool is_q = h < A.nh, is_k = h >= A.nh && h < A.nh + A.nkv;
    const bool active = live && li < lanes;
    const int pos = A.positions[t];
    it.dst = nullptr;
    if (active) {
        if (is_q) {
            it.dst = A.q_out + ((size_t)t * A.nh + h) * A.d;
        } else if (A.write_kv && A.req_of_token[t] >= 0) {
            const int page = A.block_table[(size_t)A.req_of_token[t] * A.table_stride + pos / A.page_size];
            if (page < 0 || page >= A.num_pages) {
                atomicOr(err, XB_ERR_BAD_PAGE);
            } else {
                const int g = is_k ? h - A.nh : h - A.nh - A.nkv;
                it.dst = (is_k ? A.k_cache : A.v_cache) + (((size_t)page * A.nkv + g) * A.page_size + (pos % A.page_size)) * A.d;
            }
        }
    }
    const float* nw = is_q ? A.q_w : (is_k ? A.k_w : nullptr);
    it.normed = nw && active;
    if (it.normed) {
        const float4* w4 = reinterpret_cast<const float4*>(nw);
        const float4 a0 = w4[2 * li], a1 = w4[2 * li + 1], b0 = w4[2 * (li + half_vecs)], b1 = w4[2 * (li + half_vecs) + 1];
        it.wa[0] = a0.x, it.wa[1] = a0.y, it.wa[2] = a0.z, it.wa[3] = a0.w, it.wa[4] = a1.x, it.wa[5] = a1.y, it.wa[6] = a1.z, it.wa[7] = a1.w;
        it.wb[0] = b0.x, it.wb[1] = b0.y, it.wb[2] = b0.z, it.wb[3] = b0.w, it.wb[4] = b1.x, it.wb[5] = b1.y, it.wb[6] = b1.z, it.wb[7] = b1.w;
    }
    it.rotated = A.cos_t && active && (is_q || is_k);
    // a position the table does not hold is reported; the row read instead keeps the access in bounds
    if (it.rotated && (pos < 0 || pos >= A.max_pos) && A.req_of_token[t] >= 0) atomicOr(err, XB_ERR_BAD_POSITION);
    const int tp = pos < A.max_pos ? (pos < 0 ? 0 : pos) : A.max_pos - 1;
    const int half = A.rot / 2;
    it.cr = A.cos_t + (size_t)tp * half;
    it.sr = A.sin_t + (size_t)tp * half;
    it.neox = it.rotated && !A.interleaved && A.rot == A.d;   // vector li pairs with vector li + half_vecs
    if (it.neox) {
        const float4 c0 = reinterpret_cast<const float4*>(it.cr)[2 * li], c1 = reinterpret_cast<const float4*>(it.cr)[2 * li + 1];
        const float4 s0 = reinterpret_cast<const float4*>(it.sr)[2 * li], s1 = reinterpret_cast<const float4*>(it.sr)[2 * li + 1];
        it.rc[0] = c0.x, it.rc[1] = c0.y, it.rc[2] = c0.z, it.rc[3] = c0.w, it.rc[4] = c1.x, it.rc[5] = c1.y, it.rc[6] = c1.z, it.rc[7] = c1.w;
        it.rs[0] = s0.x, it.rs[1] = s0.y, it.rs[2] = s0.z, it.rs[3] = s0.w, it.rs[4] = s1.x, it.rs[5] = s1.y, it.rs[6] = s1.z, it.rs[7] = s1.w;
    }
    return it;
}

// `a`, `b`: the lane's two vectors (zeros on a lane without work).  Every lane of the warp must call
// this, whatever its head is: the sum of squares is reduced with shuffles over the group's LPH lanes.
template <int LPH>
__device__ __forceinline__ void qk_finish(const QkArgs& A, const QkItem& it, float (&a)[8], float (&b)[8], int li) {
    const int half_vecs = A.d / 16;
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += a[e] * a[e] + b[e] * b[e];
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o, LPH);
    if (it.normed) {
        const float inv = rsqrtf(ss / (float)A.d + A.eps);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            a[e] = a[e] * inv * it.wa[e];
            b[e] = b[e] * inv * it.wb[e];
        }
    }
    if (it.neox) {
        // element i of the head pairs with i + d / 2
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float x0 = a[e], x1 = b[e];
            a[e] = x0 * it.rc[e] - x1 * it.rs[e];
            b[e] = x0 * it.rs[e] + x1 * it.rc[e];
        }
    } else if (it.rotated && A.interleaved) {
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
            const int ia = li * 8 + e, ib = (li + half_vecs) * 8 + e;  // even element indices
            if (ia < A.rot) {
                const float c = it.cr[ia / 2], s = it.sr[ia / 2], x0 = a[e], x1 = a[e + 1];
                a[e] = x0 * c - x1 * s;
                a[e + 1] = x0 * s + x1 * c;
            }
            if (ib < A.rot) {
                const float c = it.cr[ib / 2], s = it.sr[ib / 2], x0 = b[e], x1 = b[e + 1];
                b[e] = x0 * c - x1 * s;
                b[e + 1] = x0 * s + x1 * c;
            }
        }
    }
    if (it.dst) {
        reinterpret_cast<Pack8*>(it.dst)[li] = pack8(a);
        reinterpret_cast<Pack8*>(it.dst)[li + half_vecs] = pack8(b);
    }
}

}  // namespace xbqk
