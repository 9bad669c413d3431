// generated from tc_kernel_list.h by build.py
#include "../tc_inst.cuh"
TC_DEFINE_INST(tc_inst_dfma_128x128, double, TC_MATH_SIMT, 128, 128, 1, 1, 3, 1)
