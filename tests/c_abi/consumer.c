/* A plain C consumer of include/churten_b200.h: the header must compile as C11 with no
 * C++ in sight, and the library must link and answer calls that need no GPU. */
#include "churten_b200.h"

#include <stdio.h>
#include <string.h>

int main(void) {
  cb200_lr_policy policy;
  cb200_grad_parts parts;
  memset(&policy, 0, sizeof policy);
  memset(&parts, 0, sizeof parts);
  policy.kind = CB200_LR_COSINE;
  policy.t_max = 10.0;
  if (cb200_version() < 200) return 2;
  if (cb200_workspace_bytes(1024) != 256 + 4096 + 64 * 1024 + 4096) return 3;
  /* argument errors are reported before anything touches a device */
  if (cb200_scatter_rows(0, 0, -1, 1, 1, 0, 0, 0, 0, 0) != CB200_ERR_INVALID_ARGUMENT) return 4;
  if (strstr(cb200_last_error(), "must be >= 0") == 0) return 5;
  if (cb200_lr_schedule(0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 4, 0) != CB200_ERR_INVALID_ARGUMENT) return 6;
  if (cb200_adam_step_from_parts(CB200_F32, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 4, 4, 0, 0, 0, 1, 0, -1, 0, 0,
                                 0) != CB200_ERR_INVALID_ARGUMENT) return 7;
  if (cb200_copy_rows_masked(-1, 0, 0, 0, 0, 0, 0, 0, 1, 0) != CB200_ERR_INVALID_ARGUMENT) return 8;
  printf("ok %d %d %d\n", cb200_version(), (int)sizeof policy, (int)sizeof parts);
  (void)policy;
  (void)parts;
  return 0;
}
