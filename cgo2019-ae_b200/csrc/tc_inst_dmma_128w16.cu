#include "tc_inst.cuh"
TC_DEFINE_INST(tc_inst_dmma_128w16, double, TC_MATH_DMMA, 128, 128, 4, 4, 4)
