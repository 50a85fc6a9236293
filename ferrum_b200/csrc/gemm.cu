// Prefill dequant-GEMM on tcgen05 (BF16 in, BF16 out).
#include "internal.h"

int fq_launch_gemm_tc(fq_device *, const ProjectArgs &) { return FQ_ERR_UNSUPPORTED; }
