// Chooses the attention kernel for a call: the specialised decode kernels when
// the shape and representation match one, the general kernel otherwise.
#include "common.h"

#include <cstdlib>

namespace kvc {

int launch_attention_general(const AttnArgs &a, cudaStream_t stream);
int launch_attention_decode(const AttnArgs &a, cudaStream_t stream);
int launch_attention_affine(const AttnArgs &a, cudaStream_t stream);
int launch_attention_turbo(const AttnArgs &a, cudaStream_t stream);
int launch_attention_chunk_packed(const AttnArgs &a, cudaStream_t stream);
int launch_attention_chunk_tc(const AttnArgs &a, cudaStream_t stream);
int launch_attention_chunk_materialized(const AttnArgs &a, cudaStream_t stream);
int launch_attention_verify_tc_raw(const AttnArgs &a, cudaStream_t stream);

namespace {
// KVC_ATTENTION_PATH=general forces the general kernel (read once per process; used by
// tests that compare the two paths on the device from child processes).
bool force_general() {
    static const bool forced = [] {
        const char *e = std::getenv("KVC_ATTENTION_PATH");
        return e && e[0] == 'g';
    }();
    return forced;
}
}  // namespace

int launch_attention(const AttnArgs &a, cudaStream_t stream) {
    if (!force_general()) {
        int n = launch_attention_chunk_tc(a, stream);   // long chunks over raw caches: tcgen05 kernel
        if (n > 0) return n;
        n = launch_attention_verify_tc_raw(a, stream);   // verify rounds of 17 ... 64 rows per KV head over raw caches
        if (n > 0) return n;
        n = launch_attention_decode(a, stream);
        if (n > 0) return n;
        n = launch_attention_affine(a, stream);
        if (n > 0) return n;
        n = launch_attention_turbo(a, stream);
        if (n > 0) return n;
        n = launch_attention_chunk_materialized(a, stream);   // long chunks over packed caches: rows written out, then tcgen05
        if (n > 0) return n;
        n = launch_attention_chunk_packed(a, stream);
        if (n > 0) return n;
    }
    return launch_attention_general(a, stream);
}

}  // namespace kvc
