// Split-KV attention on tcgen05 (interface; kernel in splitkv_umma.cu).
#pragma once

#include "splitkv.cuh"

namespace qwb {

// Chunks this kernel takes: fewer than 64 new tokens per sequence (longer chunks go to the prefill
// kernels).  It needs arrival counters (p.cnt), i.e. the fused path that runs the append kernel.
bool splitkv_umma_usable(int n_new);
// Tokens per unit block: up to 21 (126 of the 128 tile rows).
int splitkv_umma_rb(int n_new);
// Shared-memory split for a block of rb tokens: rows of Q that are really stored, and ring slots.
void splitkv_umma_layout(int rb, int *q_rows_pad, int *nslot);
// K map: box 64 x 128 rows; V map: box 64 x 32 rows.  p.rb / p.nblk / p.G / p.ws / p.cnt must be set
// for 128-key tiles and splitkv_umma_rb().  Returns 0 or a QW_ERR_* code.
int launch_splitkv_umma(const CUtensorMap &mk, const CUtensorMap &mv, const SplitKVParams &p, bool out_is_f32,
                        cudaStream_t st, bool dependent);

}  // namespace qwb
