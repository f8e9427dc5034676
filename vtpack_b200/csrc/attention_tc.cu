// placeholder, replaced below
#include "attention.h"
namespace vtp {
int attention_tcgen05(const AttnArgs& p, cudaStream_t st) {
    (void)p; (void)st;
    return fail(VTP_ERR_UNSUPPORTED, "attention (tcgen05): not built yet");
}
}
