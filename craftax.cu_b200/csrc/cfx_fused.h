// Interface of the fused tcgen05 forward (one kernel per step) to the C-ABI layer.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace cfx {

struct FusedPlan;  // operand mirrors, tensor maps, status word; owned by the handle

struct FusedArgs {
    const uint8_t* records;
    const float* prev_terminals;
    const float* uniforms;
    float* state;  // [L][n][H]
    float* env_actions;
    int32_t* actions;
    float* logprobs;
    float* values;
    float* logits_av;
    float* r_state;
    int r_state_bf16;   // r_state holds bf16 instead of fp32
    uint64_t seed, env_offset;
    unsigned long long* step_ctr;
    int bump_step;   // 1: the kernel's last block adds one to *step_ctr when every block is done
    // 128-env tiles [tile_begin, tile_end) of the batch; tile_end = 0: all.  tile_begin must be
    // even, and tile_end even unless it is the end of the batch.
    int tile_begin = 0, tile_end = 0;
};

// Shapes the fused kernel is instantiated for.
bool fused_supported(int H, int L, int A, int precision, int game);
int fused_create(FusedPlan** out, int device, int n, int H, int L, int A, int precision,
                 float* state, int game);
// Rebuilds the operand mirrors from the fp32 arena (device pointer).
int fused_refresh(FusedPlan* plan, const float* params, cudaStream_t st);
int fused_forward(FusedPlan* plan, const FusedArgs& a, cudaStream_t st, int* launches);
// Reads and clears the device status word (non-zero = a bounded wait gave up).
int fused_check_status(FusedPlan* plan, cudaStream_t st, unsigned* status);
void fused_destroy(FusedPlan* plan);

int fused_selftest_wait_timeout(unsigned limit_ms, unsigned* status_out);

}  // namespace cfx
