// placeholder until the chunked linear-attention kernel lands
#include "../../include/attn_b200.h"
extern "C" {
int attn_b200_linear_fwd(const AttnB200LinearArgs*, void*) { return ATTN_B200_E_UNSUPPORTED; }
}
