// Expert-parallel MoE kernels that fuse the row exchange with the expert GEMMs (see the kernels below).
#include "peer.cuh"

B2_DEFINE_WAIT_SETTER(b2_moe_ep_file_set_wait_ns)
