// Python bindings, second part (quantised formats, fused collectives, MoE, MLA, drafter ops).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include "api.h"
#include "api_ext.h"

void register_ext(pybind11::module_& m) { (void)m; }
