// gtb_sample.cuh -- device-side selection over a logits row, shared by the engines of this library family
#pragma once
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace gtb {

// The k largest logits and their token ids, largest first, ties to the lower id (the candidate set of topk_sample,
// tinyllama.cpp:466-478): k rounds of a block-wide arg-max over the not-yet-taken entries.  One CTA of 1024 threads.
__global__ void __launch_bounds__(1024) k_topk(const float* __restrict__ logits, int n, int k, float* __restrict__ out_v, int32_t* __restrict__ out_i) {
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ int taken[64];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    for (int r = 0; r < k; r++) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int j = tid; j < n; j += 1024) {
            const float v = logits[j];
            bool skip = false;
            for (int q = 0; q < r; q++) skip |= (taken[q] == j);
            if (!skip && (v > best || (v == best && j < arg) || arg == 0x7fffffff)) { best = v; arg = j; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
            if (oi != 0x7fffffff && (arg == 0x7fffffff || ov > best || (ov == best && oi < arg))) { best = ov; arg = oi; }
        }
        if (lane == 0) { sv[wid] = best; si[wid] = arg; }
        __syncthreads();
        if (wid == 0) {
            best = sv[lane]; arg = si[lane];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
                if (oi != 0x7fffffff && (arg == 0x7fffffff || ov > best || (ov == best && oi < arg))) { best = ov; arg = oi; }
            }
            if (lane == 0) { taken[r] = arg; out_v[r] = best; out_i[r] = arg; }
        }
        __syncthreads();
    }
}

}  // namespace gtb
