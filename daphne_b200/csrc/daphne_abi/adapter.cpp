// Device-context registry of the adapter: one db2_context per DaphneContext (device 0, like the reference's
// CreateCUDAContext; DAPHNE_B200_DEVICE selects another device for this process).
#include <B200Adapter.h>

#include <cstdlib>
#include <map>
#include <mutex>

namespace b200 {

static std::mutex g_mu;
static std::map<DaphneContext *, db2_context *> g_ctx;

void create_context(DaphneContext *ctx) {
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_ctx.count(ctx))
        return;
    const char *dev = std::getenv("DAPHNE_B200_DEVICE");
    db2_context *c = nullptr;
    check(db2_context_create(dev ? std::atoi(dev) : 0, &c));
    g_ctx[ctx] = c;
}

db2_context *context(DaphneContext *ctx) {
    {
        std::lock_guard<std::mutex> lock(g_mu);
        auto it = g_ctx.find(ctx);
        if (it != g_ctx.end())
            return it->second;
    }
    create_context(ctx);
    std::lock_guard<std::mutex> lock(g_mu);
    return g_ctx[ctx];
}

} // namespace b200
