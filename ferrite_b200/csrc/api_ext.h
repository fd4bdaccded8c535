// C launch API, second part: quantised formats, fused compute+collective kernels, MoE, MLA, drafter ops.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifdef __cplusplus
}
#endif
