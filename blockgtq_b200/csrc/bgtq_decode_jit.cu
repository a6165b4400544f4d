// Run-time specialisation of the decode kernel for the KV heads of one layer.
//
// The kernel text (bgtq_common.cuh, bgtq_plan.h, bgtq_decode_kernel.cuh, embedded as strings by the build)
// is compiled with NVRTC behind a generated prelude that spells every head's segment list as compile-time
// constants, so the K loop of the resulting kernel is straight-line code.  NVRTC is looked up with dlopen
// (the library does not link it); the cubin is loaded through the CUDA runtime's library API.  Compiled
// kernels are cached per process by their prelude, so layers with equal bit maps share one kernel.
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "bgtq_decode_kernel.cuh"

using namespace bgtq;

namespace {

const char kSrcCommon[] =
#include "bgtq_common.cuh.str"
    ;
const char kSrcPlan[] =
#include "bgtq_plan.h.str"
    ;
const char kSrcKernel[] =
#include "bgtq_decode_kernel.cuh.str"
    ;

// ---- NVRTC through dlopen -------------------------------------------------------------------------
typedef struct _nvrtcProgram* nvrtcProgram;
struct Nvrtc {
    void* handle = nullptr;
    int (*CreateProgram)(nvrtcProgram*, const char*, const char*, int, const char* const*, const char* const*);
    int (*CompileProgram)(nvrtcProgram, int, const char* const*);
    int (*GetProgramLogSize)(nvrtcProgram, size_t*);
    int (*GetProgramLog)(nvrtcProgram, char*);
    int (*GetCUBINSize)(nvrtcProgram, size_t*);
    int (*GetCUBIN)(nvrtcProgram, char*);
    int (*DestroyProgram)(nvrtcProgram*);
};
std::mutex g_mutex;
Nvrtc g_nvrtc;
std::string g_nvrtc_path;
struct Compiled {
    std::vector<char> cubin;
    cudaLibrary_t lib = nullptr;
    cudaKernel_t kernel = nullptr;
};
std::map<std::string, Compiled> g_cache;     // prelude -> compiled kernel

bool load_nvrtc(std::string* why) {
    if (g_nvrtc.handle) return true;
    std::vector<std::string> cands;
    if (!g_nvrtc_path.empty()) cands.push_back(g_nvrtc_path);
    if (const char* e = getenv("BGTQ_NVRTC")) cands.push_back(e);
    cands.push_back("libnvrtc.so.12");
    cands.push_back("libnvrtc.so");
    // next to the CUDA runtime this library is linked against: <prefix>/lib64/ or the Python wheels' layout
    Dl_info info;
    if (dladdr(reinterpret_cast<void*>(&cudaGetDevice), &info) && info.dli_fname) {
        std::string dir(info.dli_fname);
        const size_t slash = dir.rfind('/');
        if (slash != std::string::npos) {
            dir.resize(slash);
            cands.push_back(dir + "/libnvrtc.so.12");
            cands.push_back(dir + "/../../cuda_nvrtc/lib/libnvrtc.so.12");
        }
    }
    cands.push_back("/usr/local/cuda/lib64/libnvrtc.so.12");
    cands.push_back("/usr/local/cuda/lib64/libnvrtc.so");
    void* h = nullptr;
    for (const std::string& c : cands) {
        h = dlopen(c.c_str(), RTLD_NOW | RTLD_LOCAL);
        if (h) break;
    }
    if (!h) {
        if (why) *why = "NVRTC (libnvrtc.so.12) not found; set BGTQ_NVRTC to its path";
        return false;
    }
    Nvrtc n;
    n.handle = h;
#define BGTQ_SYM(field, name) \
    *reinterpret_cast<void**>(&n.field) = dlsym(h, name); \
    if (!n.field) { if (why) *why = std::string("NVRTC symbol missing: ") + name; dlclose(h); return false; }
    BGTQ_SYM(CreateProgram, "nvrtcCreateProgram")
    BGTQ_SYM(CompileProgram, "nvrtcCompileProgram")
    BGTQ_SYM(GetProgramLogSize, "nvrtcGetProgramLogSize")
    BGTQ_SYM(GetProgramLog, "nvrtcGetProgramLog")
    BGTQ_SYM(GetCUBINSize, "nvrtcGetCUBINSize")
    BGTQ_SYM(GetCUBIN, "nvrtcGetCUBIN")
    BGTQ_SYM(DestroyProgram, "nvrtcDestroyProgram")
#undef BGTQ_SYM
    g_nvrtc = n;
    return true;
}

// The compile-time description of the layer's heads.
std::string make_prelude(const DecPlanDev& pl) {
    char buf[512];
    std::string s;
    s += "#define BGTQ_JIT 1\n#define BGTQ_HEAD_DIM 128\n";
    snprintf(buf, sizeof(buf), "#define BGTQ_JIT_VB %d\n#define BGTQ_JIT_NU 2\n", pl.v_sbits);
    s += buf;
    if (pl.row_st[0] > 0) {       // row strides fixed at compile time (and 16-byte aligned slices promised at launch)
        snprintf(buf, sizeof(buf), "#define BGTQ_JIT_STRIDES 1\n#define BGTQ_JIT_KP_ST %du\n#define BGTQ_JIT_KN_ST %du\n"
                                   "#define BGTQ_JIT_VP_ST %du\n#define BGTQ_JIT_VN_ST %du\n#define BGTQ_JIT_STAGE_OFF %uu\n",
                 pl.row_st[0], pl.row_st[1], pl.row_st[2], pl.row_st[3], kOffStagesMin + pl.lut_bytes);
        s += buf;
    }
    s += "typedef unsigned char uint8_t;\ntypedef unsigned short uint16_t;\ntypedef unsigned int uint32_t;\n"
         "typedef int int32_t;\ntypedef long long int64_t;\ntypedef unsigned long long uint64_t;\n"
         "typedef unsigned long long uintptr_t;\n"
         "namespace bgtq { namespace jit {\n"
         "struct SegC { int kind, bw, q, f16_norm, bit0, lane_bits, tbl, esh, rep_log2, ent_log2, norm_idx, step0, jv; };\n"
         "template <int H> struct Head;\n";
    for (int h = 0; h < pl.n_heads; ++h) {
        const DecHeadPlan& hp = pl.head[h];
        snprintf(buf, sizeof(buf), "template <> struct Head<%d> {\n    static constexpr int n_seg = %d;\n"
                                   "    static constexpr SegC seg[8] = {\n", h, hp.n_seg);
        s += buf;
        int step0 = 0;
        for (int g = 0; g < 8; ++g) {
            if (g < hp.n_seg) {
                const DecSeg& c = hp.seg[g];
                // lanes of a quad that hold codes of the segment: its length over the codes per lane
                const int len = (int)hp.steps[step0].end - (int)hp.steps[step0].pos;
                const int jv = c.q > 0 ? (len + c.q - 1) / c.q : 4;
                snprintf(buf, sizeof(buf), "        {%d, %d, %d, %d, %d, %d, %u, %d, %d, %d, %d, %d, %d},\n", c.kind, c.bw, c.q,
                         c.f16_norm, c.bit0, c.lane_bits, c.tbl, c.esh, c.rep_log2, c.ent_log2, c.norm_idx, step0,
                         jv < 1 ? 1 : (jv > 4 ? 4 : jv));
                step0 += (c.q + 3) / 4;
            } else {
                snprintf(buf, sizeof(buf), "        {1, 1, 0, 0, 0, 0, 0u, 0, 0, 0, 0, 0, 4},\n");
            }
            s += buf;
        }
        s += "    };\n};\n";
    }
    s += "}}\n#define BGTQ_JIT_CASES";
    for (int h = 0; h < pl.n_heads; ++h) {
        snprintf(buf, sizeof(buf), " BGTQ_JIT_CASE(%d)", h);
        s += buf;
    }
    s += "\n";
    return s;
}

// Compile one prelude to a cubin.  Runs without the lock: NVRTC is thread safe, and callers specialise the
// layers of a model from several threads.
int compile(const std::string& prelude, std::vector<char>* cubin, std::string* log) {
    const std::string src = prelude + kSrcCommon + "\n" + kSrcPlan + "\n" + kSrcKernel + "\n";
    nvrtcProgram prog = nullptr;
    if (g_nvrtc.CreateProgram(&prog, src.c_str(), "bgtq_decode_jit.cu", 0, nullptr, nullptr) != 0) return BGTQ_E_LAUNCH;
    std::vector<const char*> opts = {"--gpu-architecture=sm_100a", "--std=c++17", "-lineinfo"};
    if (getenv("BGTQ_JIT_VERBOSE")) opts.push_back("--ptxas-options=-v");
    std::vector<std::string> extra;             // BGTQ_JIT_OPTIONS: further NVRTC options, space separated
    if (const char* e = getenv("BGTQ_JIT_OPTIONS")) {
        std::string cur;
        for (const char* ch = e;; ++ch) {
            if (*ch == ' ' || *ch == 0) {
                if (!cur.empty()) extra.push_back(cur);
                cur.clear();
                if (*ch == 0) break;
            } else {
                cur.push_back(*ch);
            }
        }
    }
    for (const std::string& x : extra) opts.push_back(x.c_str());
    const int rc = g_nvrtc.CompileProgram(prog, (int)opts.size(), opts.data());
    size_t n = 0;
    if (log && g_nvrtc.GetProgramLogSize(prog, &n) == 0 && n > 1) {
        log->resize(n);
        g_nvrtc.GetProgramLog(prog, &(*log)[0]);
    }
    size_t sz = 0;
    if (rc != 0 || g_nvrtc.GetCUBINSize(prog, &sz) != 0 || sz == 0) {
        g_nvrtc.DestroyProgram(&prog);
        return BGTQ_E_LAUNCH;
    }
    cubin->resize(sz);
    g_nvrtc.GetCUBIN(prog, cubin->data());
    g_nvrtc.DestroyProgram(&prog);
    return BGTQ_OK;
}

// Compile (or find) the kernel of a prelude.  `load`: also load it into the CUDA runtime (needs a GPU).
int build(const std::string& prelude, bool load, cudaKernel_t* kernel, std::string* log) {
    bool have = false;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        std::string why;
        if (!load_nvrtc(&why)) {
            if (log) *log = why;
            return BGTQ_E_UNSUPPORTED;
        }
        auto it = g_cache.find(prelude);
        have = it != g_cache.end() && !it->second.cubin.empty();
    }
    std::vector<char> cubin;
    if (!have) {
        const int rc = compile(prelude, &cubin, log);      // two threads with the same layout both compile; one wins
        if (rc != BGTQ_OK) return rc;
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    Compiled& c = g_cache[prelude];
    if (c.cubin.empty()) c.cubin.swap(cubin);
    if (load && !c.kernel) {
        if (cudaLibraryLoadData(&c.lib, c.cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0) != cudaSuccess ||
            cudaLibraryGetKernel(&c.kernel, c.lib, "bgtq_decode_jit") != cudaSuccess) {
            cudaGetLastError();
            if (log) *log += "\nloading the compiled kernel failed";
            c.kernel = nullptr;
            return BGTQ_E_LAUNCH;
        }
    }
    if (kernel) *kernel = c.kernel;
    return BGTQ_OK;
}

void copy_log(const std::string& log, char* dst, int64_t cap) {
    if (!dst || cap <= 0) return;
    const size_t n = log.size() < (size_t)cap - 1 ? log.size() : (size_t)cap - 1;
    memcpy(dst, log.data(), n);
    dst[n] = 0;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int bgtq_jit_set_nvrtc_path(const char* path) {
    std::lock_guard<std::mutex> lock(g_mutex);
    g_nvrtc_path = path ? path : "";
    return BGTQ_OK;
}

extern "C" __attribute__((visibility("default"))) int bgtq_decode_plan_specialize(BgtqDecodePlan* plan_host,
                                                                                  int32_t compile_only, char* log,
                                                                                  int64_t log_bytes) {
    if (!plan_host) return BGTQ_E_BADARG;
    DecPlanDev pl;
    memcpy(&pl, plan_host, sizeof(pl));
    if (pl.n_heads < 1 || pl.n_heads > kMaxPlanHeads) return BGTQ_E_BADARG;
    std::string text;
    cudaKernel_t kernel = nullptr;
    const int rc = build(make_prelude(pl), compile_only == 0, &kernel, &text);
    copy_log(text, log, log_bytes);
    if (rc != BGTQ_OK) return rc;
    if (!compile_only) {
        pl.jit_kernel = kernel;
        memcpy(plan_host, &pl, sizeof(pl));
    }
    return BGTQ_OK;
}

namespace bgtq {
// Launch the specialised kernel recorded in the plan (tiles of 16 warps x 32 tokens only).
cudaError_t launch_decode_jit(const DecParams& P, dim3 grid, size_t smem, cudaStream_t stream, bool programmatic) {
    const void* fn = P.plan.jit_kernel;
    cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kDecThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    void* args[1] = {const_cast<DecParams*>(&P)};
    e = cudaLaunchKernelExC(&cfg, fn, args);
    return e == cudaSuccess ? cudaGetLastError() : e;
}
}  // namespace bgtq
