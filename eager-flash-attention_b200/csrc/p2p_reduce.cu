#include "p2p_reduce.h"

#include "host_util.h"

namespace efa {

int p2p_prepare(efa_ctx*, const efa_params&, void*)
{
    set_error("reduce=p2p is not available in this build");
    return 5;
}
int p2p_tile(efa_ctx*, const efa_params&, const efa_weights&, const void*, int, int*)
{
    set_error("reduce=p2p is not available in this build");
    return 5;
}
int p2p_finish(efa_ctx*, const efa_params&)
{
    set_error("reduce=p2p is not available in this build");
    return 5;
}
void p2p_destroy(efa_ctx*) {}

}  // namespace efa
