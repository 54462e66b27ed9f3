// Device-side categorical sampler and Philox uniform of the policy head.
#pragma once
#include <curand_kernel.h>
#include <cstdint>

namespace cfx {

// One uniform in (0, 1] for (seed, env, step): the same cuRAND device calls the
// reference issues in k_value_sample (craftax_full.cu:9733-9736).
__device__ __forceinline__ float philox_uniform(uint64_t seed, uint64_t env, uint64_t step) {
    curandStatePhilox4_32_10_t st;
    curand_init(seed ^ 0xA5A5A5A5A5A5A5A5ULL, env, step, &st);
    return curand_uniform(&st);
}

// Softmax-CDF sample with one uniform.  Operation order follows
// cf_nn_sample_action (craftax_full.cu:9147-9165): running max, p = expf(l - m)
// summed in ascending action order, first action whose running sum reaches
// u * total (default A - 1), logprob = l - m - logf(total).  A is a template
// parameter so that p[] stays in registers.
template <int A>
__device__ __forceinline__ int sample_action(const float (&logits)[A], float u, float* logprob) {
    float m = logits[0];
#pragma unroll
    for (int a = 1; a < A; a++) m = fmaxf(m, logits[a]);
    float p[A];
    float total = 0.0f;
#pragma unroll
    for (int a = 0; a < A; a++) {
        p[a] = expf(logits[a] - m);
        total += p[a];
    }
    float target = u * total, cum = 0.0f;
    int action = A - 1;
    float la = logits[A - 1];
    bool found = false;
#pragma unroll
    for (int a = 0; a < A; a++) {
        cum += p[a];
        if (!found && target <= cum) {
            action = a;
            la = logits[a];
            found = true;
        }
    }
    *logprob = la - m - logf(total);
    return action;
}

// Runtime-A variant for the stand-alone sampler entry point.
__device__ __forceinline__ int sample_action_dyn(const float* logits, int A, float u, float* logprob) {
    float m = logits[0];
    for (int a = 1; a < A; a++) m = fmaxf(m, logits[a]);
    float total = 0.0f;
    for (int a = 0; a < A; a++) total += expf(logits[a] - m);
    float target = u * total, cum = 0.0f;
    int action = A - 1;
    for (int a = 0; a < A; a++) {
        cum += expf(logits[a] - m);
        if (target <= cum) { action = a; break; }
    }
    *logprob = logits[action] - m - logf(total);
    return action;
}

}  // namespace cfx
