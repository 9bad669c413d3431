// generated from tc_kernel_list.h by build.py
#include "../tc_inst.cuh"
TC_DEFINE_INST(tc_inst_dmma_128x64_w4, double, TC_MATH_DMMA, 128, 64, 2, 2, 3, 2)
