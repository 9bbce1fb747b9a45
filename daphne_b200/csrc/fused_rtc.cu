// Row passes for chains that have no compiled-in specialisation: the kernel template of fused_ct_dev.cuh is
// instantiated for the recorded chain by the run-time compiler (NVRTC, found with dlopen), once per chain and
// process, and the resulting kernel is launched like the compiled-in ones.
//
// DAPHNE generates one kernel call per operator and knows no fused kernels, so there is no counterpart in the
// reference; the compiled-in table (fused_ct.cu) covers the chains of the benchmark pipelines, this file every other
// DaphneDSL expression that the deferred evaluation turns into a chain.
//
// The compilation takes 0.4 to 0.8 s per chain.  By default it runs on the calling thread, the first time a chain is
// evaluated.  DB2_RTC=async (or db2_rtc_set_mode(1)) moves it to a background thread: the calls that arrive meanwhile
// are served by the run-time chain interpreter of the same kernel, and the first call after the compilation has
// finished loads the binary and uses it from then on.  A process in that mode must not end while a compilation is
// running (the compiler's own static objects would be destroyed under it): db2_context_destroy and db2_rtc_wait
// wait for it.  DB2_RTC=0 switches the mechanism off, as does a missing libnvrtc (binaries kept on disk by earlier
// processes are still used then; DB2_RTC_NO_COMPILER=1 makes a process behave like that).
#include "fused.cuh"
#include "fused_ct_dev.cuh"

#include "_build/fused_rtc_src.h"

#include <dlfcn.h>
#include <sys/stat.h>
#include <sys/types.h>
#include <unistd.h>

#include <condition_variable>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace db2 {
namespace {

enum Mode { RTC_OFF = 0, RTC_ASYNC = 1, RTC_SYNC = 2 };
enum State { COMPILING = 0, COMPILED, LOADED, FAILED };

struct Nvrtc {
    typedef void *Program;
    int (*create)(Program *, const char *, const char *, int, const char *const *, const char *const *) = nullptr;
    int (*destroy)(Program *) = nullptr;
    int (*add_name)(Program, const char *) = nullptr;
    int (*compile)(Program, int, const char *const *) = nullptr;
    int (*cubin_size)(Program, size_t *) = nullptr;
    int (*cubin)(Program, char *) = nullptr;
    int (*lowered)(Program, const char *, const char **) = nullptr;
    int (*log_size)(Program, size_t *) = nullptr;
    int (*log)(Program, char *) = nullptr;
    bool ok = false;
};

const Nvrtc &nvrtc() {
    static const Nvrtc n = [] {
        Nvrtc r;
        void *h = nullptr;
        if (getenv("DB2_RTC_NO_COMPILER")) // behave like a machine without the toolkit: binaries from disk only
            return r;
        for (const char *name : {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12"})
            if ((h = dlopen(name, RTLD_NOW | RTLD_LOCAL)))
                break;
        if (!h)
            return r;
        auto sym = [&](const char *s) { return dlsym(h, s); };
        r.create = reinterpret_cast<decltype(r.create)>(sym("nvrtcCreateProgram"));
        r.destroy = reinterpret_cast<decltype(r.destroy)>(sym("nvrtcDestroyProgram"));
        r.add_name = reinterpret_cast<decltype(r.add_name)>(sym("nvrtcAddNameExpression"));
        r.compile = reinterpret_cast<decltype(r.compile)>(sym("nvrtcCompileProgram"));
        r.cubin_size = reinterpret_cast<decltype(r.cubin_size)>(sym("nvrtcGetCUBINSize"));
        r.cubin = reinterpret_cast<decltype(r.cubin)>(sym("nvrtcGetCUBIN"));
        r.lowered = reinterpret_cast<decltype(r.lowered)>(sym("nvrtcGetLoweredName"));
        r.log_size = reinterpret_cast<decltype(r.log_size)>(sym("nvrtcGetProgramLogSize"));
        r.log = reinterpret_cast<decltype(r.log)>(sym("nvrtcGetProgramLog"));
        r.ok = r.create && r.destroy && r.add_name && r.compile && r.cubin_size && r.cubin && r.lowered && r.log_size &&
               r.log;
        return r;
    }();
    return n;
}

struct Entry {
    State state = COMPILING;
    std::vector<char> cubin;
    std::string lowered, log;
    cudaLibrary_t lib = nullptr;
    cudaKernel_t kernel = nullptr;
    PerDeviceOnce attr;
};

// never destroyed: a compilation may still be running on its background thread when the process ends
struct Globals {
    std::mutex mu;
    std::condition_variable cv;
    std::map<std::string, std::shared_ptr<Entry>> cache; // by instantiation expression; entries are never removed
    int pending = 0;
    int mode = -1; // -1: not read from the environment yet
};
Globals &globals() {
    static Globals *g = new Globals;
    return *g;
}
#define g_mu (globals().mu)
#define g_cv (globals().cv)
#define g_cache (globals().cache)
#define g_pending (globals().pending)
#define g_mode (globals().mode)

int mode_locked() {
    if (g_mode < 0) {
        const char *e = getenv("DB2_RTC");
        g_mode = !e ? RTC_SYNC : (e[0] == '0' ? RTC_OFF : (strcmp(e, "async") == 0 ? RTC_ASYNC : RTC_SYNC));
    }
    return g_mode;
}

// Chain<S<op, kind, rev>...>
std::string chain_of(const FusedProgram &P) {
    std::string e = "db2::ct::Chain<";
    for (int i = 0; i < P.nsteps; i++)
        e += std::string(i ? "," : "") + "db2::ct::S<" + std::to_string(P.steps[i].op) + "," +
             std::to_string(P.steps[i].kind) + "," + (P.steps[i].reversed ? "true" : "false") + ">";
    return e + ">";
}
// fused_row_ct_kernel<Chain<...>, Taps<T<after, kind>...>, EW, AL>
std::string expression_of(const FusedProgram &P, bool aligned) {
    std::string e = "db2::ct::fused_row_ct_kernel<" + chain_of(P) + ",db2::ct::Taps<";
    for (int i = 0; i < P.ntaps; i++)
        e += std::string(i ? "," : "") + "db2::ct::T<" + std::to_string(P.taps[i].after_step) + "," +
             std::to_string(P.taps[i].kind) + ">";
    e += std::string(">,") + (P.ew_out ? "true" : "false") + "," + (aligned ? "true" : "false") + ">";
    return e;
}
// fused_col_sum_ct_kernel<Chain<...>>
std::string col_expression_of(const FusedProgram &P) { return "db2::ct::fused_col_sum_ct_kernel<" + chain_of(P) + ">"; }

// ---- binaries kept on disk ----
// DAPHNE starts a new process for every script, so a chain's kernel would be compiled again in every run.  The device
// binary is therefore also written to a directory of the user -- DB2_RTC_CACHE, else $XDG_CACHE_HOME/daphne_b200, else
// $HOME/.cache/daphne_b200; DB2_RTC_CACHE=0 (or no usable directory) switches this off -- under a name made of hashes
// of the embedded source and the instantiation, and read back from there (size and checksum verified) before the
// compiler is asked.  Files are written under a temporary name and renamed, so concurrent processes see whole files.
uint64_t fnv1a(const void *data, size_t n, uint64_t h) {
    const unsigned char *p = static_cast<const unsigned char *>(data);
    for (size_t i = 0; i < n; i++) {
        h ^= p[i];
        h *= 1099511628211ull;
    }
    return h;
}
std::string cache_dir() {
    const char *e = getenv("DB2_RTC_CACHE");
    std::string dir;
    if (e && (e[0] == '\0' || strcmp(e, "0") == 0))
        return "";
    if (e) {
        dir = e;
    } else {
        const char *x = getenv("XDG_CACHE_HOME"), *h = getenv("HOME");
        if (x && x[0] == '/')
            dir = std::string(x) + "/daphne_b200";
        else if (h && h[0] == '/') {
            dir = std::string(h) + "/.cache";
            mkdir(dir.c_str(), 0700);
            dir += "/daphne_b200";
        } else
            return "";
    }
    mkdir(dir.c_str(), 0700);
    struct stat st;
    if (stat(dir.c_str(), &st) != 0 || !S_ISDIR(st.st_mode))
        return "";
    return dir;
}
std::string cache_path(const std::string &src, const std::string &expr) {
    const std::string dir = cache_dir();
    if (dir.empty())
        return "";
    const char *what = "db2-rtc-1 sm_100a -std=c++17 -lineinfo";
    uint64_t a = fnv1a(what, strlen(what), 14695981039346656037ull), b = fnv1a(what, strlen(what), 0x9e3779b97f4a7c15ull);
    a = fnv1a(src.data(), src.size(), a);
    b = fnv1a(src.data(), src.size(), b);
    a = fnv1a(expr.data(), expr.size(), a);
    b = fnv1a(expr.data(), expr.size(), b);
    char name[64];
    snprintf(name, sizeof(name), "/%016llx%016llx.cubin", (unsigned long long)a, (unsigned long long)b);
    return dir + name;
}
struct CacheHeader {
    char magic[8]; // "DB2RTC1"
    uint64_t cubin_bytes, cubin_hash, name_bytes;
};
bool cache_load(const std::string &path, std::vector<char> *cubin, std::string *lowered) {
    FILE *f = path.empty() ? nullptr : fopen(path.c_str(), "rb");
    if (!f)
        return false;
    CacheHeader h;
    bool ok = fread(&h, sizeof(h), 1, f) == 1 && memcmp(h.magic, "DB2RTC1", 8) == 0 && h.cubin_bytes > 0 &&
              h.cubin_bytes < (64u << 20) && h.name_bytes > 0 && h.name_bytes < 65536;
    if (ok) {
        lowered->resize(h.name_bytes);
        cubin->resize(h.cubin_bytes);
        ok = fread(&(*lowered)[0], 1, h.name_bytes, f) == h.name_bytes &&
             fread(cubin->data(), 1, h.cubin_bytes, f) == h.cubin_bytes &&
             fnv1a(cubin->data(), cubin->size(), 14695981039346656037ull) == h.cubin_hash;
    }
    fclose(f);
    if (!ok) {
        cubin->clear();
        lowered->clear();
        remove(path.c_str()); // truncated or foreign file: compile again
    }
    return ok;
}
void cache_store(const std::string &path, const std::vector<char> &cubin, const std::string &lowered) {
    if (path.empty())
        return;
    const std::string tmp = path + ".tmp" + std::to_string((long long)getpid());
    FILE *f = fopen(tmp.c_str(), "wb");
    if (!f)
        return;
    CacheHeader h;
    memset(&h, 0, sizeof(h));
    memcpy(h.magic, "DB2RTC1", 8);
    h.cubin_bytes = cubin.size();
    h.cubin_hash = fnv1a(cubin.data(), cubin.size(), 14695981039346656037ull);
    h.name_bytes = lowered.size();
    const bool ok = fwrite(&h, sizeof(h), 1, f) == 1 && fwrite(lowered.data(), 1, lowered.size(), f) == lowered.size() &&
                    fwrite(cubin.data(), 1, cubin.size(), f) == cubin.size();
    if (fclose(f) != 0 || !ok || rename(tmp.c_str(), path.c_str()) != 0)
        remove(tmp.c_str());
}

// one instantiation as a cubin for sm_100a: from the directory above, else from the compiler (and then stored there);
// on failure the compiler's log is left in *log
bool compile(const std::string &expr, std::vector<char> *cubin, std::string *lowered, std::string *log) {
    std::string src;
    for (const char *piece : FUSED_RTC_SRC)
        src += piece;
    const std::string path = cache_path(src, expr);
    if (cache_load(path, cubin, lowered))
        return true;
    const Nvrtc &n = nvrtc();
    if (!n.ok) {
        *log = "libnvrtc not found";
        return false;
    }
    Nvrtc::Program prog = nullptr;
    if (n.create(&prog, src.c_str(), "fused_ct_dev.cu", 0, nullptr, nullptr) != 0) {
        *log = "nvrtcCreateProgram failed";
        return false;
    }
    const char *opts[] = {"--gpu-architecture=sm_100a", "-std=c++17", "-lineinfo"};
    bool ok = n.add_name(prog, expr.c_str()) == 0 && n.compile(prog, 3, opts) == 0;
    size_t sz = 0;
    if (!ok && n.log_size(prog, &sz) == 0 && sz > 1) {
        log->resize(sz);
        n.log(prog, &(*log)[0]);
    }
    const char *name = nullptr;
    ok = ok && n.lowered(prog, expr.c_str(), &name) == 0 && name;
    if (ok)
        *lowered = name;
    ok = ok && n.cubin_size(prog, &sz) == 0 && sz > 0;
    if (ok) {
        cubin->resize(sz);
        ok = n.cubin(prog, cubin->data()) == 0;
    }
    n.destroy(&prog);
    if (!ok && log->empty())
        *log = "the run-time compiler returned no binary";
    if (ok)
        cache_store(path, *cubin, *lowered);
    return ok;
}

void compile_entry(const std::string expr, std::shared_ptr<Entry> e) {
    std::vector<char> cubin;
    std::string lowered, log;
    const bool ok = compile(expr, &cubin, &lowered, &log);
    {
        std::lock_guard<std::mutex> lock(g_mu);
        e->cubin.swap(cubin);
        e->lowered.swap(lowered);
        e->log.swap(log);
        e->state = ok ? COMPILED : FAILED;
        g_pending--;
    }
    g_cv.notify_all();
}

} // namespace

namespace {
// The loaded kernel of an instantiation, or null: not ready yet (its compilation is started if it has not been), failed
// or switched off.
std::shared_ptr<Entry> kernel_of(const std::string &expr) {
    std::shared_ptr<Entry> e;
    std::unique_lock<std::mutex> lock(g_mu);
    const int mode = mode_locked();
    if (mode == RTC_OFF)
        return nullptr;
    auto it = g_cache.find(expr);
    if (it == g_cache.end()) {
        e = std::make_shared<Entry>();
        g_cache[expr] = e;
        g_pending++;
        lock.unlock();
        if (mode == RTC_SYNC)
            compile_entry(expr, e);
        else
            std::thread(compile_entry, expr, e).detach();
        lock.lock();
    } else {
        e = it->second;
    }
    if (e->state == COMPILED) { // first call after the compiler finished: load the binary
        cudaError_t err = cudaLibraryLoadData(&e->lib, e->cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0);
        if (err == cudaSuccess)
            err = cudaLibraryGetKernel(&e->kernel, e->lib, e->lowered.c_str());
        if (err != cudaSuccess) {
            cudaGetLastError();
            e->log = std::string("loading the compiled kernel failed: ") + cudaGetErrorString(err);
            e->state = FAILED; // (a binary that came from disk is not trusted again: its file is removed)
            std::string src;
            for (const char *piece : FUSED_RTC_SRC)
                src += piece;
            const std::string path = cache_path(src, expr);
            if (!path.empty())
                remove(path.c_str());
        } else {
            e->state = LOADED;
            std::vector<char>().swap(e->cubin);
        }
    }
    return e->state == LOADED ? e : nullptr;
}
} // namespace

// Launches the run-time compiled specialisation of P's chain if it is ready (true; *rc is the launch's result).
// Otherwise starts its compilation, if that has not happened yet, and returns false: the caller runs the interpreter.
bool fused_row_pass_rtc(const FusedProgram &P, bool aligned, cudaStream_t st, int *rc) {
    std::shared_ptr<Entry> e = kernel_of(expression_of(P, aligned));
    if (!e)
        return false;
    using namespace ct;
    const size_t smem = (size_t)(WARPS * 2 * WR * CK + P.smem_elems + 2 * FUSED_MAX_STEPS) * sizeof(double) + 256;
    const int64_t nblocks = ((P.rows + WR - 1) / WR + WARPS - 1) / WARPS;
    const int64_t cap = (int64_t)sm_count() * RowCtasPerSm<AnyChain>::value; // the same for every chain
    const int grid = (int)(nblocks < cap ? nblocks : cap);
    const void *fn = reinterpret_cast<const void *>(e->kernel);
    if (e->attr.need()) {
        const cudaError_t err = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
        if (err != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        e->attr.mark();
    }
    void *args[] = {const_cast<FusedProgram *>(&P)};
    const cudaError_t err = cudaLaunchKernel(fn, dim3((unsigned)grid), dim3(RT), args, smem, st);
    if (err != cudaSuccess) {
        cudaGetLastError();
        *rc = set_error(DB2_ECUDA, "launch of a run-time compiled row pass failed: %s", cudaGetErrorString(err));
        return true;
    }
    *rc = after_launch("fused_row_ct_kernel (run-time compiled)");
    return true;
}

// The same for the column sums / means of a chain; until the kernel exists the caller runs the general column pass.
bool fused_col_pass_rtc(const FusedProgram &P, int mean, void *res, void *scratch, cudaStream_t st, int *rc) {
    std::shared_ptr<Entry> e = kernel_of(col_expression_of(P));
    if (!e)
        return false;
    unsigned grid[2], block[2];
    fused_col_geometry(P, grid, block);
    double *part = static_cast<double *>(scratch);
    void *args[] = {const_cast<FusedProgram *>(&P), &part};
    const cudaError_t err = cudaLaunchKernel(reinterpret_cast<const void *>(e->kernel), dim3(grid[0], grid[1]),
                                             dim3(block[0], block[1]), args, 0, st);
    if (err != cudaSuccess) {
        cudaGetLastError();
        *rc = set_error(DB2_ECUDA, "launch of a run-time compiled column pass failed: %s", cudaGetErrorString(err));
        return true;
    }
    *rc = after_launch("fused_col_sum_ct_kernel (run-time compiled)");
    if (*rc == DB2_OK)
        *rc = fused_col_finish(P, grid[0], mean, res, scratch, st);
    return true;
}

} // namespace db2

using namespace db2;

extern "C" {

int db2_rtc_set_mode(int mode) {
    DB2_CHECK(mode >= RTC_OFF && mode <= RTC_SYNC, DB2_EINVAL, "mode must be 0 (off), 1 (background) or 2 (blocking)");
    std::lock_guard<std::mutex> lock(g_mu);
    g_mode = mode;
    return DB2_OK;
}

int db2_rtc_wait(void) {
    std::unique_lock<std::mutex> lock(g_mu);
    g_cv.wait(lock, [] { return g_pending == 0; });
    return DB2_OK;
}

int db2_rtc_counts(int *ready, int *pending, int *failed) {
    std::lock_guard<std::mutex> lock(g_mu);
    int r = 0, f = 0;
    for (const auto &kv : g_cache) {
        r += kv.second->state == COMPILED || kv.second->state == LOADED;
        f += kv.second->state == FAILED;
    }
    if (ready)
        *ready = r;
    if (pending)
        *pending = g_pending;
    if (failed)
        *failed = f;
    return DB2_OK;
}

int db2_rtc_compile(const int *ops, const int *kinds, const int *reversed, int nsteps, const int *tap_after,
                    const int *tap_kinds, int ntaps, int ew, size_t *binary_bytes) {
    const bool column_pass = ntaps < 0; // column sums of the chain instead of row aggregations
    if (column_pass)
        ntaps = 0;
    DB2_CHECK(nsteps >= 0 && nsteps <= FUSED_MAX_STEPS && ntaps <= FUSED_MAX_AGGS, DB2_EINVAL,
              "at most %d steps and %d aggregations", FUSED_MAX_STEPS, FUSED_MAX_AGGS);
    DB2_CHECK((nsteps == 0 || (ops && kinds && reversed)) && (ntaps == 0 || (tap_after && tap_kinds)), DB2_EINVAL,
              "null argument");
    FusedProgram P;
    memset(&P, 0, sizeof(P));
    P.nsteps = nsteps;
    P.ntaps = ntaps;
    for (int i = 0; i < nsteps; i++) {
        DB2_CHECK(ops[i] >= 0 && ops[i] < FO_COUNT && kinds[i] >= FK_MATRIX && kinds[i] <= FK_UNARY, DB2_EINVAL,
                  "step %d: unknown operation or operand kind", i);
        P.steps[i].op = ops[i];
        P.steps[i].kind = kinds[i];
        P.steps[i].reversed = reversed[i] != 0;
    }
    for (int i = 0; i < ntaps; i++) {
        DB2_CHECK(tap_after[i] >= 0 && tap_after[i] <= nsteps && tap_kinds[i] >= FT_SUM && tap_kinds[i] <= FT_MEAN,
                  DB2_EINVAL, "aggregation %d: unknown kind or position", i);
        P.taps[i].after_step = tap_after[i];
        P.taps[i].kind = tap_kinds[i];
    }
    P.ew_out = (ew & 1) ? &P : nullptr; // only its presence matters here
    std::vector<char> cubin;
    std::string lowered, log;
    if (!compile(column_pass ? col_expression_of(P) : expression_of(P, (ew & 2) == 0), &cubin, &lowered, &log))
        return set_error(DB2_EUNSUPPORTED, "run-time compilation failed: %.900s", log.c_str());
    if (binary_bytes)
        *binary_bytes = cubin.size();
    return DB2_OK;
}

} // extern "C"
