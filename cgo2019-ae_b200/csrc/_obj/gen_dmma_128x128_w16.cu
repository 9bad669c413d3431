// generated from tc_kernel_list.h by build.py
#include "../tc_inst.cuh"
TC_DEFINE_INST(tc_inst_dmma_128x128_w16, double, TC_MATH_DMMA, 128, 128, 4, 4, 4, 1)
