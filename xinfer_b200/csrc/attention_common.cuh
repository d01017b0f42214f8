// What the attention kernels of both families share.
#pragma once
#include "common.cuh"

// Which token the z-th "small" token of the batch is: tokens of entries that bring at most
// dec_max tokens, in batch order (direct != 0: every token of the batch is one).  -1 if there is none.
__device__ __forceinline__ int small_token(int z, const int* __restrict__ q_start, int num_entries, int dec_max, int direct) {
    if (direct) return z < q_start[num_entries] ? z : -1;
    int acc = 0;
    for (int b = 0; b < num_entries; ++b) {
        const int n = q_start[b + 1] - q_start[b];
        if (n > 0 && n <= dec_max) {
            if (z < acc + n) return q_start[b] + z - acc;
            acc += n;
        }
    }
    return -1;
}
