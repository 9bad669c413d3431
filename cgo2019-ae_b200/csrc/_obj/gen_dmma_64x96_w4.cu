// generated from tc_kernel_list.h by build.py
#include "../tc_inst.cuh"
TC_DEFINE_INST(tc_inst_dmma_64x96_w4, double, TC_MATH_DMMA, 64, 96, 2, 2, 3, 3)
