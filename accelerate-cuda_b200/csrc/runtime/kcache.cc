/*
 * kcache.cc -- from functor source to a loaded kernel: source assembly,
 * hashing, the two-level (memory, disk) kernel cache, the nvcc worker pool
 * and per-context module loading.
 *
 * Replaces build/build1/compile/link/compileFlags/enqueueProcess of
 * Data/Array/Accelerate/CUDA/Compile.hs:439-660 and the KernelTable of
 * Data/Array/Accelerate/CUDA/Persistent.hs:77-378.  Differences that matter:
 *   - the key is a hash of (arch, contents of the skeleton headers, assembled
 *     source, extra flags) instead of (compute capability, MD5 of the
 *     generated source) (Compile.hs:565, Persistent.hs:175), so editing a
 *     skeleton header invalidates old cubins;
 *   - the on-disk cache is one file per key, written with an atomic rename;
 *     there is no count-prefixed index file to corrupt (Persistent.hs:352-378);
 *   - a second, read-only cache directory next to the library holds cubins
 *     compiled at build time.
 */
#include <dirent.h>
#include <dlfcn.h>
#include <fcntl.h>
#include <spawn.h>
#include <sys/stat.h>
#include <sys/wait.h>
#include <unistd.h>

#include <algorithm>
#include <cstdlib>
#include <fstream>
#include <sstream>
#include <thread>

#include "common.h"

extern char **environ;

namespace accb_rt {

static const SkeletonDesc kSkeletons[] = {
    {"map", "map.cuh", "ACCB_INSTANTIATE_MAP", SK_MAP},
    {"fold_all", "fold.cuh", "ACCB_INSTANTIATE_FOLD_ALL", SK_FOLD_ALL},
    {"fold_dim", "fold.cuh", "ACCB_INSTANTIATE_FOLD_DIM", SK_FOLD_DIM},
    {"fold_seg", "fold.cuh", "ACCB_INSTANTIATE_FOLD_SEG", SK_FOLD_SEG},
    {"scan", "scan.cuh", "ACCB_INSTANTIATE_SCAN", SK_SCAN},
    {"permute", "permute.cuh", "ACCB_INSTANTIATE_PERMUTE", SK_PERMUTE},
    {"permute_smem", "permute.cuh", "ACCB_INSTANTIATE_PERMUTE_SMEM", SK_PERMUTE_SMEM},
    {"stencil", "stencil.cuh", "ACCB_INSTANTIATE_STENCIL", SK_STENCIL},
    {"stencil2", "stencil.cuh", "ACCB_INSTANTIATE_STENCIL2", SK_STENCIL2},
    {"stencil3", "stencil3.cuh", "ACCB_INSTANTIATE_STENCIL3", SK_STENCIL3}, /* stencil over a rank-3 array */
};

const SkeletonDesc *find_skeleton(const char *name) {
    if (!name) return nullptr;
    for (const auto &s : kSkeletons)
        if (strcmp(s.name, name) == 0) return &s;
    return nullptr;
}

/* ---- paths ---- */
static std::string lib_dir() {
    Dl_info info;
    if (dladdr((void *)&find_skeleton, &info) && info.dli_fname) {
        std::string p = info.dli_fname;
        size_t slash = p.rfind('/');
        return slash == std::string::npos ? "." : p.substr(0, slash);
    }
    return ".";
}

std::string include_dir() {
    if (const char *e = getenv("ACCB_INCLUDE_DIR")) return e;
    return lib_dir() + "/csrc";
}

static const char *kArch = "sm_100a";

std::string preseed_cache_dir() { return lib_dir() + "/kcache/" + kArch; }

std::string default_cache_dir() {
    if (const char *e = getenv("ACCB_CACHE_DIR")) return std::string(e) + "/" + kArch;
    const char *home = getenv("HOME");
    return std::string(home ? home : "/tmp") + "/.accelerate/accelerate-b200-" + accb_version() + "/cache/" + kArch;
}

static void mkdirs(const std::string &path) {
    for (size_t i = 1; i <= path.size(); ++i)
        if (i == path.size() || path[i] == '/') mkdir(path.substr(0, i).c_str(), 0755);
}

static bool read_file(const std::string &path, std::string *out) {
    std::ifstream f(path, std::ios::binary);
    if (!f) return false;
    std::ostringstream ss;
    ss << f.rdbuf();
    *out = ss.str();
    return true;
}

/* ---- hashing: two independent 64-bit FNV-1a style lanes -> 128-bit hex ---- */
struct Hash128 {
    uint64_t a = 0xcbf29ce484222325ull, b = 0x9ae16a3b2f90404full;
    void add(const void *data, size_t n) {
        const unsigned char *p = static_cast<const unsigned char *>(data);
        for (size_t i = 0; i < n; ++i) {
            a = (a ^ p[i]) * 0x100000001b3ull;
            b = (b ^ (p[i] + 0x9e)) * 0xc6a4a7935bd1e995ull;
            b ^= b >> 29;
        }
    }
    void add(const std::string &s) {
        add(s.data(), s.size());
        add("\x1f", 1);
    }
    std::string hex() const {
        char buf[40];
        snprintf(buf, sizeof buf, "%016llx%016llx", (unsigned long long)a, (unsigned long long)b);
        return buf;
    }
};

/* hash of every skeleton / support header: the "skeleton library version" */
static const std::string &library_fingerprint() {
    static std::string fp;
    static std::once_flag once;
    std::call_once(once, [] {
        Hash128 h;
        const std::string inc = include_dir();
        for (const char *sub : {"/cubits", "/skeletons"}) {
            std::vector<std::string> names;
            if (DIR *d = opendir((inc + sub).c_str())) {
                while (dirent *e = readdir(d))
                    if (e->d_name[0] != '.') names.push_back(e->d_name);
                closedir(d);
            }
            std::sort(names.begin(), names.end());
            for (const auto &n : names) {
                std::string body;
                if (read_file(inc + sub + "/" + n, &body)) {
                    h.add(n);
                    h.add(body);
                }
            }
        }
        fp = h.hex();
    });
    return fp;
}

std::string make_source(const SkeletonDesc *sk, const char *src, const char *name) {
    std::ostringstream s;
    s << "#include \"skeletons/" << sk->header << "\"\n" << src << "\n" << sk->macro << "(" << name << ")\n";
    return s.str();
}

std::string cache_key(const SkeletonDesc *sk, const char *src, const char *name, const char *flags) {
    Hash128 h;
    h.add(std::string(kArch));
    h.add(library_fingerprint());
    h.add(make_source(sk, src, name));
    h.add(std::string(flags ? flags : ""));
    return h.hex();
}

/* ---- nvcc worker pool: at most one compiler per host core in flight
 * (the MSem of Compile.hs:620-622) ---- */
struct Semaphore {
    std::mutex mu;
    std::condition_variable cv;
    int avail;
    explicit Semaphore(int n) : avail(n) {}
    void acquire() {
        std::unique_lock<std::mutex> l(mu);
        cv.wait(l, [&] { return avail > 0; });
        --avail;
    }
    void release() {
        std::lock_guard<std::mutex> l(mu);
        ++avail;
        cv.notify_one();
    }
};
static Semaphore &nvcc_slots() {
    static Semaphore s(std::max(1u, std::thread::hardware_concurrency()));
    return s;
}

static std::vector<std::string> split_flags(const char *flags) {
    std::vector<std::string> out;
    std::istringstream ss(flags ? flags : "");
    std::string tok;
    while (ss >> tok) out.push_back(tok);
    return out;
}

static int run_nvcc(const std::string &cu, const std::string &cubin, const char *flags, std::string *log) {
    if (inject_failure("nvcc")) {
        *log = "injected nvcc failure";
        return ACCB_ECOMPILE;
    }
    const char *nvcc = getenv("ACCB_NVCC");
    std::string nvcc_path = nvcc ? nvcc : "nvcc";
    if (!nvcc && access("/usr/local/cuda/bin/nvcc", X_OK) == 0) nvcc_path = "/usr/local/cuda/bin/nvcc";
    const std::string inc = "-I" + include_dir();
    std::vector<std::string> args = {nvcc_path, "-arch=sm_100a", "-cubin", "-O3", "-std=c++17", "-DNDEBUG",
                                     "-m64",    "-lineinfo",     inc};
    for (auto &f : split_flags(flags)) args.push_back(f);
    args.push_back("-o");
    args.push_back(cubin);
    args.push_back(cu);
    std::vector<char *> argv;
    for (auto &a : args) argv.push_back(const_cast<char *>(a.c_str()));
    argv.push_back(nullptr);

    const std::string logfile = cu + ".log";
    posix_spawn_file_actions_t fa;
    posix_spawn_file_actions_init(&fa);
    posix_spawn_file_actions_addopen(&fa, 1, logfile.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
    posix_spawn_file_actions_adddup2(&fa, 1, 2);
    pid_t pid;
    nvcc_slots().acquire();
    int rc = posix_spawnp(&pid, nvcc_path.c_str(), &fa, nullptr, argv.data(), environ);
    int status = -1;
    if (rc == 0) waitpid(pid, &status, 0);
    nvcc_slots().release();
    posix_spawn_file_actions_destroy(&fa);
    read_file(logfile, log);
    unlink(logfile.c_str());
    if (rc != 0) {
        *log = "cannot start " + nvcc_path + ": " + strerror(rc);
        return ACCB_ECOMPILE;
    }
    if (!WIFEXITED(status) || WEXITSTATUS(status) != 0) return ACCB_ECOMPILE;
    return ACCB_OK;
}

/* process-wide first-level cache: key -> cubin bytes */
static std::mutex g_mem_mu;
static std::unordered_map<std::string, std::shared_ptr<std::string>> g_mem;

CompileResult compile_or_load(const std::string &key, const std::string &source, const char *flags,
                              const char *cache_dir_override) {
    CompileResult r;
    {
        std::lock_guard<std::mutex> l(g_mem_mu);
        auto it = g_mem.find(key);
        if (it != g_mem.end()) {
            r.cubin = *it->second;
            r.source = 1;
            return r;
        }
    }
    const std::string user_dir = cache_dir_override ? std::string(cache_dir_override) + "/" + kArch : default_cache_dir();
    const bool flush = getenv("ACCB_FLUSH_CACHE") != nullptr;
    if (!flush) {
        for (const std::string &dir : {user_dir, preseed_cache_dir()}) {
            if (inject_failure("cache_io")) break;
            if (read_file(dir + "/" + key + ".cubin", &r.cubin) && !r.cubin.empty()) {
                r.source = 2;
                std::lock_guard<std::mutex> l(g_mem_mu);
                g_mem[key] = std::make_shared<std::string>(r.cubin);
                return r;
            }
        }
    }
    /* miss: compile in a private temporary directory, then move into place */
    mkdirs(user_dir);
    char tmpl[] = "/tmp/accb-XXXXXX";
    const char *tmp = mkdtemp(tmpl);
    if (!tmp) {
        r.status = ACCB_EIO;
        r.log = "mkdtemp failed";
        return r;
    }
    const std::string cu = std::string(tmp) + "/" + key + ".cu";
    const std::string cubin = std::string(tmp) + "/" + key + ".cubin";
    {
        std::ofstream f(cu);
        f << source;
    }
    r.status = run_nvcc(cu, cubin, flags, &r.log);
    if (trace_enabled("cc"))
        fprintf(stderr, "[accb cc] nvcc %s -> %s\n%s", key.c_str(), r.status == ACCB_OK ? "ok" : "FAILED", r.log.c_str());
    if (r.status == ACCB_OK && !read_file(cubin, &r.cubin)) {
        r.status = ACCB_EIO;
        r.log = "compiler produced no cubin";
    }
    if (r.status == ACCB_OK) {
        r.source = 3;
        /* persist: write beside the final name, then rename (atomic on one filesystem) */
        const std::string fin = user_dir + "/" + key + ".cubin";
        const std::string part = fin + ".part." + std::to_string((long)getpid());
        std::ofstream f(part, std::ios::binary);
        f.write(r.cubin.data(), (std::streamsize)r.cubin.size());
        f.close();
        if (!f || rename(part.c_str(), fin.c_str()) != 0) unlink(part.c_str()); /* cache stays cold; not fatal */
        std::lock_guard<std::mutex> l(g_mem_mu);
        g_mem[key] = std::make_shared<std::string>(r.cubin);
    }
    if (!getenv("ACCB_KEEP_SOURCE")) {
        unlink(cu.c_str());
        unlink(cubin.c_str());
        rmdir(tmp);
    }
    return r;
}

/* process-wide kernel table: one accb_kernel per key */
static std::mutex g_table_mu;
static std::unordered_map<std::string, accb_kernel *> g_table;

int get_function(accb_context *ctx, accb_kernel *k, const char *entry, CUfunction *fn, KernelMeta *meta) {
    const CompileResult &r = k->result.get(); /* blocks until the compiler is done: the lazy link */
    if (r.status != ACCB_OK) return fail(ctx, r.status, "kernel %s failed to compile:\n%s", k->key.c_str(), r.log.c_str());
    std::lock_guard<std::mutex> l(k->mu);
    LoadedModule &m = k->loaded[ctx];
    const Driver &d = driver();
    if (!m.mod) {
        int st = check_cu(ctx, d.ModuleLoadData(&m.mod, r.cubin.data()), "cuModuleLoadData");
        if (st != ACCB_OK) {
            k->loaded.erase(ctx);
            return st;
        }
        /* ask the module for its launch metadata */
        CUfunction q;
        int *dev = nullptr;
        st = check_cu(ctx, d.ModuleGetFunction(&q, m.mod, "accb_meta_query"), "accb_meta_query lookup");
        if (st == ACCB_OK) st = check_cuda(ctx, cudaMalloc((void **)&dev, sizeof(m.meta.v)), "cudaMalloc");
        if (st == ACCB_OK) {
            void *args[] = {&dev};
            st = check_cu(ctx, d.LaunchKernel(q, 1, 1, 1, 1, 1, 1, 0, nullptr, args, nullptr), "accb_meta_query");
        }
        if (st == ACCB_OK)
            st = check_cuda(ctx, cudaMemcpy(m.meta.v, dev, sizeof(m.meta.v), cudaMemcpyDeviceToHost), "metadata readback");
        if (dev) cudaFree(dev);
        if (st != ACCB_OK) {
            d.ModuleUnload(m.mod);
            k->loaded.erase(ctx);
            return st;
        }
        if (r.source == 1) ctx->mem_hits++;
        else if (r.source == 2) ctx->disk_hits++;
        else ctx->compiles++;
    }
    auto it = m.fn.find(entry);
    if (it == m.fn.end()) {
        CUfunction f;
        if (d.ModuleGetFunction(&f, m.mod, entry) != CUDA_SUCCESS)
            return fail(ctx, ACCB_ENOTFOUND, "kernel %s has no entry point '%s'", k->key.c_str(), entry);
        /* allow the full 227 KB of dynamic shared memory */
        d.FuncSetAttribute(f, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, 227 * 1024 - 1024);
        it = m.fn.emplace(entry, f).first;
    }
    *fn = it->second;
    if (meta) *meta = m.meta;
    return ACCB_OK;
}

/* A context is going away: unload the modules loaded for it and drop their entries, which are keyed by the
 * context's address -- a later context may be allocated at the same address, on another device. */
void forget_context(accb_context *ctx) {
    std::lock_guard<std::mutex> l(g_table_mu);
    for (auto &kv : g_table) {
        accb_kernel *k = kv.second;
        std::lock_guard<std::mutex> lk(k->mu);
        auto it = k->loaded.find(ctx);
        if (it == k->loaded.end()) continue;
        if (it->second.mod) driver().ModuleUnload(it->second.mod);
        k->loaded.erase(it);
    }
}

}  // namespace accb_rt

using namespace accb_rt;

extern "C" {

int accb_kernel_get(accb_context *ctx, const char *skeleton, const char *functor_src, const char *functor_name,
                    const char *nvcc_flags, accb_kernel **kernel) {
    if (!kernel || !functor_src || !functor_name) return fail(ctx, ACCB_EINVAL, "null argument");
    const SkeletonDesc *sk = find_skeleton(skeleton);
    if (!sk) return fail(ctx, ACCB_EINVAL, "unknown skeleton '%s'", skeleton ? skeleton : "(null)");
    const std::string key = cache_key(sk, functor_src, functor_name, nvcc_flags);
    std::lock_guard<std::mutex> l(g_table_mu);
    auto it = g_table.find(key);
    if (it != g_table.end()) {
        it->second->refs++;
        *kernel = it->second;
        return ACCB_OK;
    }
    accb_kernel *k = new accb_kernel;
    k->key = key;
    k->skeleton = sk->id;
    const std::string source = make_source(sk, functor_src, functor_name);
    const std::string flags = nvcc_flags ? nvcc_flags : "";
    k->result = std::async(std::launch::async, [key, source, flags] {
                    return compile_or_load(key, source, flags.c_str(), nullptr);
                }).share();
    k->refs++; /* the table's own reference */
    g_table[key] = k;
    *kernel = k;
    return ACCB_OK;
}

int accb_kernel_wait(accb_context *ctx, accb_kernel *kernel) {
    if (!kernel) return fail(ctx, ACCB_EINVAL, "null kernel");
    const CompileResult &r = kernel->result.get();
    if (r.status != ACCB_OK) return fail(ctx, r.status, "kernel %s failed to compile:\n%s", kernel->key.c_str(), r.log.c_str());
    return ACCB_OK;
}

int accb_kernel_info(accb_context *ctx, accb_kernel *kernel, const char *entry, int *regs, int *static_smem,
                     int *block, int *blocks_per_sm) {
    if (!ctx || !kernel || !entry) return fail(ctx, ACCB_EINVAL, "null argument");
    std::lock_guard<std::recursive_mutex> lock_(ctx->mu);
    CtxGuard g(ctx);
    CUfunction fn;
    KernelMeta meta;
    int st = get_function(ctx, kernel, entry, &fn, &meta);
    if (st != ACCB_OK) return st;
    const Driver &d = driver();
    int r = 0, s = 0, mt = 0;
    d.FuncGetAttribute(&r, CU_FUNC_ATTRIBUTE_NUM_REGS, fn);
    d.FuncGetAttribute(&s, CU_FUNC_ATTRIBUTE_SHARED_SIZE_BYTES, fn);
    d.FuncGetAttribute(&mt, CU_FUNC_ATTRIBUTE_MAX_THREADS_PER_BLOCK, fn);
    const int cta = meta.v[1] > 0 ? meta.v[1] : mt;
    if (regs) *regs = r;
    if (static_smem) *static_smem = s;
    if (block) *block = cta;
    if (blocks_per_sm) {
        st = occupancy(ctx, fn, cta, 0, blocks_per_sm);
        if (st != ACCB_OK) return st;
    }
    return ACCB_OK;
}

int accb_kernel_release(accb_context *ctx, accb_kernel *kernel) {
    (void)ctx;
    if (!kernel) return ACCB_OK;
    kernel->refs--; /* the table keeps its reference: kernels live as long as the process,
                       like the reference's global kernel table (State.hs:111-132) */
    return ACCB_OK;
}

int accb_kernel_precompile(const char *skeleton, const char *functor_src, const char *functor_name,
                           const char *nvcc_flags, const char *cache_dir, char *log, size_t log_bytes) {
    const SkeletonDesc *sk = find_skeleton(skeleton);
    if (!sk || !functor_src || !functor_name) return fail(nullptr, ACCB_EINVAL, "bad argument");
    const std::string key = cache_key(sk, functor_src, functor_name, nvcc_flags);
    CompileResult r = compile_or_load(key, make_source(sk, functor_src, functor_name), nvcc_flags, cache_dir);
    if (log && log_bytes) snprintf(log, log_bytes, "%s", r.log.c_str());
    if (r.status != ACCB_OK) return fail(nullptr, r.status, "precompile of %s failed:\n%s", key.c_str(), r.log.c_str());
    if (cache_dir && r.source != 3) {
        /* found elsewhere (memory or the other directory): make sure this directory has it too */
        const std::string dir = std::string(cache_dir) + "/" + kArch;
        mkdirs(dir);
        std::ofstream f(dir + "/" + key + ".cubin", std::ios::binary);
        f.write(r.cubin.data(), (std::streamsize)r.cubin.size());
    }
    return ACCB_OK;
}

int accb_kernel_key(const char *skeleton, const char *functor_src, const char *functor_name, const char *nvcc_flags,
                    char *key, size_t key_bytes) {
    const SkeletonDesc *sk = find_skeleton(skeleton);
    if (!sk || !functor_src || !functor_name || !key || key_bytes < 33) return fail(nullptr, ACCB_EINVAL, "bad argument");
    snprintf(key, key_bytes, "%s", cache_key(sk, functor_src, functor_name, nvcc_flags).c_str());
    return ACCB_OK;
}

int accb_cache_flush(accb_context *ctx) {
    {
        std::lock_guard<std::mutex> l(g_mem_mu);
        g_mem.clear();
    }
    const std::string dir = default_cache_dir();
    if (DIR *d = opendir(dir.c_str())) {
        while (dirent *e = readdir(d)) {
            const std::string n = e->d_name;
            if (n.size() > 6 && n.substr(n.size() - 6) == ".cubin") unlink((dir + "/" + n).c_str());
        }
        closedir(d);
    }
    (void)ctx;
    return ACCB_OK;
}

int accb_cache_stats(accb_context *ctx, size_t *mem_hits, size_t *disk_hits, size_t *compiles) {
    if (!ctx) return fail(nullptr, ACCB_EINVAL, "null context");
    std::lock_guard<std::recursive_mutex> lock_(ctx->mu);
    if (mem_hits) *mem_hits = ctx->mem_hits;
    if (disk_hits) *disk_hits = ctx->disk_hits;
    if (compiles) *compiles = ctx->compiles;
    return ACCB_OK;
}

} /* extern "C" */
