// tcgen05 tensor-core contractions (precision tiers PBG_PREC_TF32X3 / PBG_PREC_TF32).
#include "pbg_common.cuh"

bool pbg_tc_available() { return false; }
int launch_score_tc(const WaveDims &, const WaveBatches &, const WaveBufs &, int, cudaStream_t) { return 0; }
int launch_grad_tc(const WaveDims &, const WaveBatches &, const WaveBufs &, int, cudaStream_t) { return 0; }
