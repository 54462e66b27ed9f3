// Launchers of the strict-fp32 kernels and of the stand-alone stages.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace cfx {

struct StrictArgs {
    int n, H, L, A;
    int game = 0;           // CFX_GAME_FULL or CFX_GAME_CLASSIC (148-byte records, gather encoder)
    const float* params;    // fp32 arena
    const float* gates_t;   // [L][H][3H] transposed gate matrices
    const uint8_t* records;
    const float* prev_terminals;
    const float* uniforms;
    float* state;           // [L][n][H]
    float* scratch_h[2];    // [n][H] each
    float* logits_av;       // [n][A+1]
    float* r_state;
    int r_state_bf16 = 0;   // r_state holds bf16 instead of fp32
    float* env_actions;
    int32_t* actions;
    float* logprobs;
    float* values;
    uint64_t seed, env_offset;
    const unsigned long long* step_ctr;
};

int strict_forward(const StrictArgs& a, cudaStream_t st, int* launches);
int launch_expand(const uint8_t* rec, float* out, int n, cudaStream_t st);
int launch_classic_expand(const uint8_t* rec, float* out, int n, cudaStream_t st);
int launch_done_to_terminals(const int8_t* done, float* out, int n, cudaStream_t st);
int launch_sample(const float* logits, int ld, int A, const float* u, uint64_t seed,
                  uint64_t env_offset, const unsigned long long* step_ctr, int n,
                  float* env_actions, int32_t* actions, float* logprobs, float* values,
                  cudaStream_t st);
int launch_uniforms(uint64_t seed, uint64_t env_offset, uint64_t step, int n, float* u, cudaStream_t st);
int launch_bump(unsigned long long* ctr, cudaStream_t st);
int launch_transpose_gates(const float* W, float* Wt, int H, int L, cudaStream_t st);
int launch_init_uniform(float* w, int count, float bound, uint64_t seed, int subseq, cudaStream_t st);

}  // namespace cfx
