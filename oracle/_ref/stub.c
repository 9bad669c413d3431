/* generated: the drivers' call into the generated GPU entry does nothing here */
void sd_t_d2_fusion_() {}
