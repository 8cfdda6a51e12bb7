// Interface of the fast rotate + quantize kernel (codec_fast.cu).
#pragma once
#include "common.cuh"

namespace omni {

struct FastQuantArgs {
    const void* x; int64_t xs_b, xs_h, xs_t;
    const float* codebooks; int cb_per_head;
    const int32_t* user_ids; int32_t user_id;
    int64_t B; int H; int64_t T;
    uint8_t* nib; uint8_t* qjl; float* norms;
    int64_t os_b, os_h; const int64_t* out_offsets; int64_t out_offset;
    const uint32_t* g_rows;
};

// true when the fast kernel covers this call (shape, alignment); the caller falls back otherwise
bool fast_quantize_eligible(const FastQuantArgs& a, int dtype);
int32_t launch_fast_quantize(const FastQuantArgs& a, int dtype, int rotate, cudaStream_t st);

// stand-alone rotation of n_rows contiguous rows (16-byte aligned buffers)
int32_t launch_fast_rotate(const void* x, void* y, int64_t n_rows, int dtype, cudaStream_t st);

}  // namespace omni
