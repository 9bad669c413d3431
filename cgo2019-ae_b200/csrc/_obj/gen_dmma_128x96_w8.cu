// generated from tc_kernel_list.h by build.py
#include "../tc_inst.cuh"
TC_DEFINE_INST(tc_inst_dmma_128x96_w8, double, TC_MATH_DMMA, 128, 96, 4, 2, 3, 1)
