#include "prefill_umma.cuh"

namespace qwb {
bool prefill_umma_supported(int) { return false; }
int launch_prefill_umma(const PrefillCall &, cudaStream_t, int *n) { *n = 0; return 2; }
}  // namespace qwb
