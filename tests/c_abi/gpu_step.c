/* One Adam step through the C ABI from a program that knows nothing of PyTorch: device memory
 * from the CUDA runtime, plain pointers in, a status code out.  Three replicas of 10 parameters
 * (ragged: the element-wise kernel), the middle one frozen.  Exit code 0 = all checks passed. */
#include <cuda_runtime_api.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "churten_b200.h"

#define ROWS 3
#define LEN 10
#define CHECK(call)                                                          \
  do {                                                                       \
    cudaError_t e_ = (call);                                                 \
    if (e_ != cudaSuccess) {                                                 \
      printf("CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__); \
      return 10;                                                             \
    }                                                                        \
  } while (0)

static void* to_device(const void* host, size_t bytes) {
  void* dev = 0;
  if (cudaMalloc(&dev, bytes) != cudaSuccess) return 0;
  if (cudaMemcpy(dev, host, bytes, cudaMemcpyHostToDevice) != cudaSuccess) return 0;
  return dev;
}

int main(void) {
  float p[ROWS][LEN], g[ROWS][LEN], zeros[ROWS][LEN], steps[ROWS] = {0, 4, 0};
  const float lr[ROWS] = {1e-2f, 1e-2f, 3e-3f}, beta1[ROWS] = {0.9f, 0.9f, 0.8f};
  const float beta2[ROWS] = {0.999f, 0.999f, 0.99f}, eps[ROWS] = {1e-8f, 1e-8f, 1e-8f};
  const float wd[ROWS] = {0.0f, 0.0f, 0.0f};
  const uint8_t mask[ROWS] = {1, 0, 1};
  memset(zeros, 0, sizeof zeros);
  for (int r = 0; r < ROWS; ++r) {
    for (int i = 0; i < LEN; ++i) {
      p[r][i] = 0.5f + 0.01f * (float)(r * LEN + i);
      g[r][i] = (i % 2 ? -1.0f : 1.0f) * 0.1f * (float)(i + 1);
    }
  }
  void *dp = to_device(p, sizeof p), *dg = to_device(g, sizeof g), *dm = to_device(zeros, sizeof zeros),
       *dv = to_device(zeros, sizeof zeros), *dsteps = to_device(steps, sizeof steps),
       *dlr = to_device(lr, sizeof lr), *db1 = to_device(beta1, sizeof beta1),
       *db2 = to_device(beta2, sizeof beta2), *deps = to_device(eps, sizeof eps),
       *dwd = to_device(wd, sizeof wd), *dmask = to_device(mask, sizeof mask);
  if (!dp || !dg || !dm || !dv || !dsteps || !dlr || !db1 || !db2 || !deps || !dwd || !dmask) return 11;
  void* workspace = 0;
  const size_t workspace_bytes = cb200_workspace_bytes(ROWS);
  CHECK(cudaMalloc(&workspace, workspace_bytes));

  const int rc = cb200_adam_step(CB200_F32, dp, dg, dm, dv, 0, dsteps, dlr, db1, db2, deps, dwd,
                                 (const uint8_t*)dmask, ROWS, LEN, 0, /*amsgrad=*/0, /*maximize=*/0,
                                 /*decoupled_weight_decay=*/1, /*steps_already_bumped=*/0,
                                 /*active_rows_hint=*/-1, workspace, workspace_bytes, /*stream=*/0);
  if (rc != CB200_OK) {
    printf("cb200_adam_step: %d %s\n", rc, cb200_last_error());
    return 12;
  }
  float out[ROWS][LEN], out_steps[ROWS], out_m[ROWS][LEN];
  CHECK(cudaDeviceSynchronize());
  CHECK(cudaMemcpy(out, dp, sizeof out, cudaMemcpyDeviceToHost));
  CHECK(cudaMemcpy(out_m, dm, sizeof out_m, cudaMemcpyDeviceToHost));
  CHECK(cudaMemcpy(out_steps, dsteps, sizeof out_steps, cudaMemcpyDeviceToHost));

  if (out_steps[0] != 1.0f || out_steps[1] != 4.0f || out_steps[2] != 1.0f) return 13;
  if (memcmp(out[1], p[1], sizeof p[1]) != 0) return 14; /* the frozen replica: same bytes */
  for (int i = 0; i < LEN; ++i) {
    if (out_m[1][i] != 0.0f) return 15;
  }
  for (int r = 0; r < ROWS; r += 2) { /* first Adam step of the active replicas, in double */
    for (int i = 0; i < LEN; ++i) {
      const double grad = g[r][i], m = (1.0 - beta1[r]) * grad, v = (1.0 - beta2[r]) * grad * grad;
      const double m_hat = m / (1.0 - beta1[r]), v_hat = v / (1.0 - beta2[r]);
      const double want = p[r][i] - lr[r] * m_hat / (sqrt(v_hat) + eps[r]);
      if (fabs(out[r][i] - want) > 1e-6 * fabs(want)) {
        printf("row %d element %d: got %.9g, want %.9g\n", r, i, out[r][i], want);
        return 16;
      }
      if (fabs(out_m[r][i] - m) > 1e-6 * fabs(m)) return 17;
    }
  }
  printf("ok\n");
  return 0;
}
