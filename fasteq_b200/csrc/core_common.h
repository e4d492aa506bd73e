// Host-side helpers shared by the translation units of libfasteq_b200_core.
#pragma once
#include <cuda_runtime.h>
namespace fasteq {
extern thread_local char g_cuda_err[256];
int cuda_fail(cudaError_t e);
}
