// generated from tc_kernel_list.h by build.py
#include "../tc_inst.cuh"
TC_DEFINE_INST(tc_inst_dmma_64x64_w4, double, TC_MATH_DMMA, 64, 64, 2, 2, 3, 4)
