// placeholder until the MLA decode kernels land
#include "../../include/attn_b200.h"
extern "C" {
int attn_b200_mla_plan(const AttnB200MlaShape*, int32_t, int32_t*) { return ATTN_B200_E_UNSUPPORTED; }
int64_t attn_b200_mla_workspace_bytes(const AttnB200MlaShape*, int32_t) { return 0; }
int attn_b200_mla_decode(const AttnB200MlaArgs*, void*) { return ATTN_B200_E_UNSUPPORTED; }
}
