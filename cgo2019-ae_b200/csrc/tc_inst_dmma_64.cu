#include "tc_inst.cuh"
TC_DEFINE_INST(tc_inst_dmma_64, double, TC_MATH_DMMA, 64, 64, 2, 2, 4)
