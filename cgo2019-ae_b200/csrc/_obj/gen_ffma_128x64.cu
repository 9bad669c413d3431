// generated from tc_kernel_list.h by build.py
#include "../tc_inst.cuh"
TC_DEFINE_INST(tc_inst_ffma_128x64, float, TC_MATH_SIMT, 128, 64, 1, 1, 4, 3)
