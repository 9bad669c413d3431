/* A caller written the way the reference's drivers are (cogent/drivers/tccg/code_main_tccg_02.c:17-83):
 * C89, the entry reached through an implicit declaration, sizes from argv, host tensors from malloc.
 * Reads C, A, B as raw doubles from files, calls sd_t_d2_fusion_, writes C back. */
#include <stdio.h>
#include <stdlib.h>

static double* slurp(const char* path, long n) {
  FILE* f = fopen(path, "rb");
  double* p = (double*)malloc(sizeof(double) * n);
  if (!f || !p || fread(p, sizeof(double), n, f) != (size_t)n) { fprintf(stderr, "cannot read %s\n", path); exit(2); }
  fclose(f);
  return p;
}

int main(int argc, char** argv) {
  int size_idx_a, size_idx_b, size_idx_c, size_idx_d;
  long size_C, size_A, size_B;
  double *host_C, *host_A, *host_B;
  FILE* f;
  if (argc != 9) return 2;
  size_idx_a = atoi(argv[1]); size_idx_b = atoi(argv[2]); size_idx_c = atoi(argv[3]); size_idx_d = atoi(argv[4]);
  size_C = (long)size_idx_a * size_idx_b * size_idx_c;
  size_A = (long)size_idx_d * size_idx_c * size_idx_a;
  size_B = (long)size_idx_b * size_idx_d;
  host_C = slurp(argv[5], size_C); host_A = slurp(argv[6], size_A); host_B = slurp(argv[7], size_B);
  sd_t_d2_fusion_(size_idx_a, size_idx_b, size_idx_c, size_idx_d, host_C, host_A, host_B, 1, -1);
  f = fopen(argv[8], "wb");
  if (!f || fwrite(host_C, sizeof(double), size_C, f) != (size_t)size_C) return 3;
  fclose(f);
  free(host_C); free(host_A); free(host_B);
  return 0;
}
