/*
 * TEST INFRASTRUCTURE - stand-in header used only when the reference is
 * compiled into oracle/_ref as the parity checker and CPU baseline.
 *
 * mlx/data/core/image/ImageTransform.cpp:7-10 includes <stb_image_resize2.h>
 * (nothings/stb, not vendored by the reference and absent here).  This stand-in
 * declares the one symbol that file calls, with the argument order of the call
 * at mlx/data/core/image/ImageTransform.cpp:49-58, and forwards it to the
 * restatement in oracle/resize_restatement.h.  Everything else compiled into
 * oracle/_ref is the reference's own source.
 */
#ifndef MLXD_ORACLE_SHIM_STB_IMAGE_RESIZE2_H
#define MLXD_ORACLE_SHIM_STB_IMAGE_RESIZE2_H

#include "../resize_restatement.h"

typedef int stbir_pixel_layout;

static inline unsigned char* stbir_resize_uint8_linear(
    const unsigned char* input, int input_w, int input_h, int input_stride,
    unsigned char* output, int output_w, int output_h, int output_stride,
    stbir_pixel_layout channels) {
  if (input_stride != 0 || output_stride != 0) {
    return 0; /* the reference only ever passes packed rows */
  }
  if (!mlxd_oracle_resize_u8(input, input_w, input_h, output, output_w, output_h, (int)channels)) {
    return 0;
  }
  return output;
}

#endif
