// Shared definitions of the chunked KDA kernels.
#pragma once
#include <cuda_bf16.h>
namespace hippo {
typedef __nv_bfloat16 bf16;
constexpr int KDA_CHUNK = 64;
}
