// The warp-level decode attention kernels with the per-user low-rank query update folded into their prologue
// (reference kernels/fused_attention.py:166-191 applies the update inside its attention kernel as well).
// Same source as qattn_mma.cu, compiled with the update switched on; launch_mma hands calls that carry an update
// to launch_mma_lora.
#define OMNI_MMA_LORA 1
#include "qattn_mma.cu"
