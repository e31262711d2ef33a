/* prefill.cu -- placeholder until the tcgen05 kernel lands. */
#include "ctx.h"
int hy3a_launch_prefill(hy3a_ctx *ctx, int, int, int, int, const void *, float *, size_t) {
    return hy3a_fail(ctx, HY3A_ESTATE, "prefill: kernel not built into this library");
}
