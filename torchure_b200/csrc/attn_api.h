// Host-callable launchers of the tcgen05 flash-attention kernels (attention_sm100.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
