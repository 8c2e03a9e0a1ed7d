from . import wanx2_1_t2v, wanx2_1_t2v_opt
