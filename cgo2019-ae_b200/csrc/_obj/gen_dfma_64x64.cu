// generated from tc_kernel_list.h by build.py
#include "../tc_inst.cuh"
TC_DEFINE_INST(tc_inst_dfma_64x64, double, TC_MATH_SIMT, 64, 64, 1, 1, 4, 1)
