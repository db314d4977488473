// conv2d as an implicit GEMM on the tensor cores (TF32).  Placeholder until the kernel lands:
// reports UNIMPLEMENTED so that fb200_conv2d runs the strict direct kernel.
#include "common.cuh"

extern "C" int fb200_conv2d_tcgen05(const void*, const void*, const void*, void*,
                                    const fb200_conv2d_params*, int, const fb200_epilogue*,
                                    fb200_stream) {
  return FB200_UNIMPLEMENTED;
}
