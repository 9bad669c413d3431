// generated from tc_kernel_list.h by build.py
#include "../tc_inst.cuh"
TC_DEFINE_INST(tc_inst_dmma_128x128_w8, double, TC_MATH_DMMA, 128, 128, 2, 4, 4, 1)
