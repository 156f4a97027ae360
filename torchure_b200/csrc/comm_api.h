// Host-callable launchers of the NVLink collective kernels (comm.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
