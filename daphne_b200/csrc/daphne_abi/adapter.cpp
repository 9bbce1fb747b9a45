// Device-context registry of the adapter: one device group per DaphneContext.  The reference's CreateCUDAContext makes
// one context, for device 0 (src/runtime/local/kernels/CUDA/CreateCUDAContext.cpp:4-9); here the group holds one
// context per device of DAPHNE_B200_DEVICES (comma-separated; default: every visible device; DAPHNE_B200_DEVICE=<d>
// is the short form for a single device).  Stand-alone kernels run on the group's first context; the scheduler
// (vectorized_pipeline.cpp) binds each of its worker threads to one context of the group for the duration of its task.
#include <B200Adapter.h>

#include <cstdlib>
#include <map>
#include <mutex>

namespace b200 {

static std::mutex g_mu;
static std::map<DaphneContext *, db2_group *> g_groups;
static thread_local db2_context *tls_context = nullptr;

void create_context(DaphneContext *ctx) {
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_groups.count(ctx))
        return;
    db2_group *g = nullptr;
    const char *one = std::getenv("DAPHNE_B200_DEVICE");
    if (one && !std::getenv("DAPHNE_B200_DEVICES")) {
        const int dev = std::atoi(one);
        check(db2_group_create(&dev, 1, &g));
    } else {
        check(db2_group_create(nullptr, 0, &g));
    }
    g_groups[ctx] = g;
}

db2_group *group(DaphneContext *ctx) {
    {
        std::lock_guard<std::mutex> lock(g_mu);
        auto it = g_groups.find(ctx);
        if (it != g_groups.end())
            return it->second;
    }
    create_context(ctx);
    std::lock_guard<std::mutex> lock(g_mu);
    return g_groups[ctx];
}

db2_context *context(DaphneContext *ctx) {
    if (tls_context)
        return tls_context;
    db2_context *c = nullptr;
    check(db2_group_context(group(ctx), 0, &c));
    return c;
}

ThreadContext::ThreadContext(db2_context *c) : prev(tls_context) { tls_context = c; }
ThreadContext::~ThreadContext() { tls_context = prev; }

std::mutex &mdo_mutex(const void *mdo) {
    static std::mutex stripes[64];
    return stripes[(reinterpret_cast<uintptr_t>(mdo) >> 6) % 64];
}

} // namespace b200
