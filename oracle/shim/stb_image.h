/*
 * TEST INFRASTRUCTURE - stand-in for the image decoder header that
 * mlx/data/core/image/ImageSTBI.cpp:6-7 includes.  File decoding is outside the
 * transform-and-batch path; every entry point reports failure.
 */
#ifndef MLXD_ORACLE_SHIM_STB_IMAGE_H
#define MLXD_ORACLE_SHIM_STB_IMAGE_H

typedef unsigned char stbi_uc;

static inline stbi_uc* stbi_load(const char*, int*, int*, int*, int) { return 0; }
static inline stbi_uc* stbi_load_from_memory(const stbi_uc*, int, int*, int*, int*, int) { return 0; }
static inline int stbi_info(const char*, int*, int*, int*) { return 0; }
static inline int stbi_info_from_memory(const stbi_uc*, int, int*, int*, int*) { return 0; }
static inline void stbi_image_free(void*) {}

#endif
