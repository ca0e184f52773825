/*
 * C11 client of libhodu_b200: proves that include/hodu_b200.h is valid C and that the ABI is
 * callable without Python.  Built by tests/test_c_abi.py with
 *   gcc -std=c11 -Wall -Wextra -Werror -pedantic
 *
 *   abi_smoke host   no device needed: version, error strings, argument errors
 *   abi_smoke gpu    one hodu_b200_dot call per kernel family on device 0, checked against a
 *                    plain C triple loop (inputs are small integers, so every sum is exact in
 *                    f32 and in bf16's 8-bit mantissa products)
 * Exit code 0 = every check passed; otherwise the failing check is printed.
 */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <cuda_runtime_api.h>

#include "hodu_b200.h"

#define CHECK(cond, ...)                      \
  do {                                        \
    if (!(cond)) {                            \
      fprintf(stderr, "FAILED %s: ", #cond);  \
      fprintf(stderr, __VA_ARGS__);           \
      fprintf(stderr, "\n");                  \
      return 1;                               \
    }                                         \
  } while (0)

static int host_checks(void) {
  CHECK(hodu_b200_version() == 100, "version %d", hodu_b200_version());
  CHECK(strcmp(hodu_b200_strerror(HODU_B200_OK), "ok") == 0, "strerror(0) = %s", hodu_b200_strerror(0));
  CHECK(strcmp(hodu_b200_strerror(HODU_B200_ERR_INVALID_INPUT), "invalid input") == 0, "strerror(-2)");
  /* metadata of the wrong length is refused before any device is touched */
  size_t md[8] = {2, 3, 2, 3, 1, 2, 1, 0};
  float x[6] = {0};
  int r = hodu_b200_dot(0, NULL, HODU_DTYPE_F32, x, x, x, md, 8);
  CHECK(r == HODU_B200_ERR_INVALID_INPUT, "short dot metadata returned %d", r);
  CHECK(strstr(hodu_b200_last_error_message(), "metadata length") != NULL, "message: %s", hodu_b200_last_error_message());
  r = hodu_b200_force_path(99);
  CHECK(r == HODU_B200_ERR_INVALID_INPUT, "force_path(99) returned %d", r);
  CHECK(HODU_B200_STATIC_SCRATCH_BYTES == (32u << 20), "static scratch size");
  printf("host checks ok\n");
  return 0;
}

static uint16_t bf16_of_small_int(int v) { /* exact for |v| <= 256 */
  float f = (float)v;
  uint32_t u;
  memcpy(&u, &f, 4);
  return (uint16_t)(u >> 16);
}
static float f32_of_bf16(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static int gpu_checks(void) {
  CHECK(cudaSetDevice(0) == cudaSuccess, "no CUDA device 0");
  CHECK(hodu_b200_init(0) == 0, "init: %s", hodu_b200_last_error_message());
  /* 1. f32, the reference's first dot known answer shape: [2,3] . [3,2] (generic kernel) */
  {
    const float a[6] = {1, 2, 3, 4, 5, 6}, b[6] = {7, 8, 9, 10, 11, 12};
    const size_t md[9] = {2, 3, 2, 3, 1, 2, 1, 0, 0};
    float *da, *db, *dc, c[4];
    CHECK(cudaMalloc((void**)&da, sizeof a) == cudaSuccess && cudaMalloc((void**)&db, sizeof b) == cudaSuccess &&
              cudaMalloc((void**)&dc, sizeof c) == cudaSuccess, "cudaMalloc");
    cudaMemcpy(da, a, sizeof a, cudaMemcpyHostToDevice);
    cudaMemcpy(db, b, sizeof b, cudaMemcpyHostToDevice);
    int r = hodu_b200_dot(0, NULL, HODU_DTYPE_F32, da, db, dc, md, 9);
    CHECK(r == 0, "dot f32: %s", hodu_b200_last_error_message());
    uint32_t word = 1;
    CHECK(hodu_b200_last_status(0, &word) == 0 && word == 0, "status word %u", word);
    cudaMemcpy(c, dc, sizeof c, cudaMemcpyDeviceToHost);
    CHECK(c[0] == 58 && c[1] == 64 && c[2] == 139 && c[3] == 154, "got %g %g %g %g", c[0], c[1], c[2], c[3]);
    cudaFree(da); cudaFree(db); cudaFree(dc);
  }
  /* 2. bf16 256 x 256 x 256 on the tensor-core path, entries in {-2..2}: every sum exact */
  {
    enum { D = 256 };
    uint16_t* a = malloc(sizeof(uint16_t) * D * D);
    uint16_t* b = malloc(sizeof(uint16_t) * D * D);
    uint16_t* c = malloc(sizeof(uint16_t) * D * D);
    CHECK(a && b && c, "malloc");
    uint32_t s = 12345;
    for (int i = 0; i < D * D; ++i) {
      s = s * 1664525u + 1013904223u;
      a[i] = bf16_of_small_int((int)((s >> 16) % 5) - 2);
      s = s * 1664525u + 1013904223u;
      b[i] = bf16_of_small_int((int)((s >> 16) % 3) - 1);
    }
    const size_t md[9] = {D, D, D, D, 1, D, 1, 0, 0};
    void *da, *db, *dc;
    CHECK(cudaMalloc(&da, 2 * D * D) == cudaSuccess && cudaMalloc(&db, 2 * D * D) == cudaSuccess &&
              cudaMalloc(&dc, 2 * D * D) == cudaSuccess, "cudaMalloc");
    cudaMemcpy(da, a, 2 * D * D, cudaMemcpyHostToDevice);
    cudaMemcpy(db, b, 2 * D * D, cudaMemcpyHostToDevice);
    uint64_t before = hodu_b200_launch_count();
    int r = hodu_b200_dot(0, NULL, HODU_DTYPE_BF16, da, db, dc, md, 9);
    CHECK(r == 0, "dot bf16: %s", hodu_b200_last_error_message());
    CHECK(hodu_b200_last_path() == HODU_B200_PATH_TENSOR, "path %d", hodu_b200_last_path());
    CHECK(hodu_b200_launch_count() == before + 1, "launch count");
    uint32_t word = 1;
    CHECK(hodu_b200_last_status(0, &word) == 0 && word == 0, "status word %u", word);
    cudaMemcpy(c, dc, 2 * D * D, cudaMemcpyDeviceToHost);
    for (int i = 0; i < D; ++i)
      for (int j = 0; j < D; ++j) {
        float want = 0;
        for (int k = 0; k < D; ++k) want += f32_of_bf16(a[i * D + k]) * f32_of_bf16(b[k * D + j]);
        /* |want| <= 512 and integral: representable in bf16 only up to 256 exactly, so compare
           after the same rounding the kernel applies (round to nearest even to 8 bits) */
        float got = f32_of_bf16(c[i * D + j]);
        float tol = want < 0 ? -want / 128 : want / 128;
        CHECK(got - want <= tol && want - got <= tol, "C[%d][%d] = %g, want %g", i, j, got, want);
      }
    cudaFree(da); cudaFree(db); cudaFree(dc);
    free(a); free(b); free(c);
  }
  hodu_b200_shutdown(0);
  printf("gpu checks ok\n");
  return 0;
}

int main(int argc, char** argv) {
  if (argc == 2 && strcmp(argv[1], "host") == 0) return host_checks();
  if (argc == 2 && strcmp(argv[1], "gpu") == 0) return host_checks() || gpu_checks();
  fprintf(stderr, "usage: %s host|gpu\n", argv[0]);
  return 2;
}
