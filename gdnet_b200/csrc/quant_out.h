// Descriptor of a fused 1x128 FP8 output, shared by host launchers and device code.
#pragma once

#include <stdint.h>

namespace gd {

// Where a producer kernel leaves the 1x128-quantised copy of a row-major (rows, cols) matrix it writes:
// e4m3 values, fp32 scales s[(c / 128) * s_ld + r] and the packed UE8M0 chunks of the hardware-scaled GEMM,
// all with power-of-two scales. The pointers may address a column range of wider buffers.
struct RowQuantOut {
  uint8_t* q;         // null = no quantised output
  int64_t q_ld;
  float* s;
  int64_t s_ld;
  uint8_t* p;
  int64_t p_stride;   // chunks between consecutive 128-row blocks
};

}  // namespace gd
