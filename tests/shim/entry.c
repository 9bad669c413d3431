/* The translation unit a maintainer links instead of the generated temp__NN.cu object. */
#include "tc_b200_shim.h"
TC_DEFINE_SD_T_D2_FUSION_4("t3 [a,16,b,16,c,16] += sum(d,16) * t2 [d,c,a] * v2 [b,d];", double, TC_F64)
