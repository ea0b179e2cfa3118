// step_params.h -- the parameters of a decode step that live in device memory, so that a captured CUDA graph can be
// replayed for every position and the greedy sampler's kernel can advance them without a host round trip.
#pragma once
#include <stdint.h>

namespace lmrs {

struct StepParams {
    uint32_t token;      // decode: token id; serial prefill: row index into the staged embeddings
    uint32_t pos;        // position of this step
    uint32_t mask_base;  // Gemma window quirk: the reference tests `pos - t` with the BATCH start pos
    uint32_t seq;        //   (src/transformer.rs:525); decode passes pos.  seq: launch number (grid-barrier base)
};

}  // namespace lmrs
