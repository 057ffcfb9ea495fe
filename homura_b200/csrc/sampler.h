// Argument block of the device-side sampler (sampler.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/homura_b200.h"

namespace hm {

constexpr int SAMPLER_MAX_K = 1024;  // candidates the device sampler gathers and sorts

struct SamplerArgs {
    const float* logits;  // [batch][ld_logits]
    int ld_logits, n;     // row stride and vocabulary size
    hm_sampling cfg;
    // generated tokens of every sequence: either rows of the engine's token history ...
    uint32_t* hist;        // [batch][hist_stride] token at every position (NULL: use `generated`)
    int hist_stride;
    const int32_t* gen_start;  // [batch] position of the first generated token
    const int32_t* pos;        // [batch] current length; the sampled token is also stored at hist[pos]
    // ... or one explicit list (standalone call, batch 1)
    const uint32_t* generated;
    int n_generated;
    unsigned long long* rng;  // [batch] xorshift64 state, advanced by one draw
    float* scaled;            // scratch [batch][n]
    int* count;               // scratch [batch][n], all zero on entry and on exit
    uint32_t* next_tok;       // [batch] out
    uint32_t* feed_tok;       // [batch] optional: input token of the next decode step
    int* overflow;            // [batch] out, required when top_k is outside 1..SAMPLER_MAX_K: 1 = the top-p prefix did not end
                              // inside the SAMPLER_MAX_K largest candidates (token and RNG untouched; sample this row on the host)
};

cudaError_t launch_sample(const SamplerArgs& a, int batch, cudaStream_t st);

}  // namespace hm
