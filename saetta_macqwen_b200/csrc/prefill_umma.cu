// placeholder until the tcgen05 kernel lands
#include "host.hpp"
namespace saetta {
int prefill_configure(int) { return SAETTA_OK; }
int launch_prefill(const PrefillArgs &, uint32_t *, cudaStream_t) { return fail(SAETTA_ERR_UNSUPPORTED, "prefill kernel not built"); }
}
