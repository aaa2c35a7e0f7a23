// Device copies of the IQ code books (generated header, see include/gen_iq_tables.py).  Each
// translation unit that includes this file gets its own copy in global memory of the tables it
// uses; the matmul kernels stage what they need into shared memory because lanes index the tables
// with unrelated values.
#pragma once
#define GGUF_B200_TABLE_QUAL static __device__ const
#include "../../include/gguf_b200_iq_tables.h"

namespace gguf_b200 {
#define d_iq2xxs_grid gguf_b200_iq2xxs_grid
#define d_ksigns_iq2xs gguf_b200_ksigns_iq2xs
#define d_kvalues_iq4nl gguf_b200_kvalues_iq4nl
#define d_iq2xs_grid gguf_b200_iq2xs_grid
#define d_iq2s_grid gguf_b200_iq2s_grid
#define d_iq3xxs_grid gguf_b200_iq3xxs_grid
#define d_iq3s_grid gguf_b200_iq3s_grid
#define d_iq1s_grid gguf_b200_iq1s_grid
}  // namespace gguf_b200
