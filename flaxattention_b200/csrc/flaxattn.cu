// Host side of the C ABI declared in include/flaxattn.h, plus the kernels that do not
// depend on a score_mod / mask_mod (table compaction, backward preprocess, decode combine).
//
// Kernels that embed user mods are compiled at run time: the mod fragment is placed in
// front of a kernel template from the kernels/ directory, compiled for sm_100a with
// NVRTC, cached in memory per module and on disk per content hash, and loaded through the
// context-independent library API of the CUDA runtime.
#include <cuda_runtime.h>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <nvrtc.h>

#include <dlfcn.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/flaxattn.h"
#include "kernels/fa_params.h"

#ifndef FA_STATIC_SCRATCH_BYTES
#define FA_STATIC_SCRATCH_BYTES (16u << 20)
#endif

namespace {

thread_local std::string g_err;
int fail(int code, const std::string& msg) {
  g_err = msg;
  return code;
}
#define FA_CUDA_CHECK(expr)                                                                       \
  do {                                                                                            \
    cudaError_t e_ = (expr);                                                                      \
    if (e_ != cudaSuccess)                                                                        \
      return fail(FA_ECUDA, std::string(#expr) + ": " + cudaGetErrorName(e_) + ": " + cudaGetErrorString(e_)); \
  } while (0)

std::mutex g_mu;
std::string g_kernel_dir, g_cache_dir;
bool g_cache_dir_set = false;
std::atomic<int> g_compile_count{0};

// ---- small utilities -------------------------------------------------------------------
uint64_t fnv1a(const std::string& s, uint64_t seed) {
  uint64_t h = seed;
  for (unsigned char c : s) {
    h ^= c;
    h *= 1099511628211ull;
  }
  return h;
}
std::string hash_hex(const std::string& s) {
  char buf[40];
  snprintf(buf, sizeof buf, "%016llx%016llx", (unsigned long long)fnv1a(s, 1469598103934665603ull),
           (unsigned long long)fnv1a(s, 0x9e3779b97f4a7c15ull));
  return buf;
}
bool read_file(const std::string& path, std::string& out) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return false;
  std::ostringstream ss;
  ss << f.rdbuf();
  out = ss.str();
  return true;
}
void mkdirs(const std::string& path) {
  std::string cur;
  for (size_t i = 0; i < path.size(); ++i) {
    cur.push_back(path[i]);
    if (path[i] == '/' || i + 1 == path.size()) mkdir(cur.c_str(), 0755);
  }
}
std::string kernel_dir() {
  if (!g_kernel_dir.empty()) return g_kernel_dir;
  if (const char* e = getenv("FLAXATTN_KERNEL_DIR")) return g_kernel_dir = e;
  Dl_info info;
  if (dladdr((void*)&fnv1a, &info) && info.dli_fname) {
    std::string p = info.dli_fname;
    size_t k = p.rfind('/');
    const std::string base = k == std::string::npos ? std::string(".") : p.substr(0, k);
    struct stat sb;
    g_kernel_dir = base + "/kernels";
    if (stat(g_kernel_dir.c_str(), &sb) != 0) g_kernel_dir = base + "/csrc/kernels";
  } else {
    g_kernel_dir = "kernels";
  }
  return g_kernel_dir;
}
std::string cache_dir() {
  if (g_cache_dir_set) return g_cache_dir;
  g_cache_dir_set = true;
  if (const char* e = getenv("FLAXATTN_CACHE_DIR")) return g_cache_dir = e;
  const char* home = getenv("HOME");
  g_cache_dir = std::string(home ? home : "/tmp") + "/.cache/flaxattn_b200";
  return g_cache_dir;
}

const char* const kTemplateFiles[] = {"fa_params.h", "fa_common.cuh", "fa_fwd.cuh", "fa_bwd.cuh",
                                      "fa_decode.cuh", "fa_blockmask.cuh", "fa_sm100.cuh", "fa_fwd_tc.cuh", "fa_bwd_tc.cuh", "fa_selftest.cuh"};
std::string g_templates_hash;
int templates_hash(std::string& out) {
  if (g_templates_hash.empty()) {
    std::string all;
    for (const char* f : kTemplateFiles) {
      std::string s;
      if (read_file(kernel_dir() + "/" + f, s)) all += s;
      all += "\n--\n";
    }
    if (all.size() < 200) return fail(FA_ECOMPILE, "kernel templates not found in '" + kernel_dir() + "'");
    g_templates_hash = hash_hex(all);
  }
  out = g_templates_hash;
  return FA_OK;
}

// ---- run-time compilation --------------------------------------------------------------
int nvrtc_compile(const std::string& src, const std::vector<std::string>& opts, std::string& cubin) {
  nvrtcProgram prog;
  nvrtcResult r = nvrtcCreateProgram(&prog, src.c_str(), "flaxattn_kernel.cu", 0, nullptr, nullptr);
  if (r != NVRTC_SUCCESS) return fail(FA_ECOMPILE, std::string("nvrtcCreateProgram: ") + nvrtcGetErrorString(r));
  std::vector<const char*> o;
  for (auto& s : opts) o.push_back(s.c_str());
  r = nvrtcCompileProgram(prog, (int)o.size(), o.data());
  if (r != NVRTC_SUCCESS) {
    size_t n = 0;
    nvrtcGetProgramLogSize(prog, &n);
    std::string log(n, '\0');
    if (n) nvrtcGetProgramLog(prog, &log[0]);
    nvrtcDestroyProgram(&prog);
    return fail(FA_ECOMPILE, std::string("kernel compilation failed: ") + nvrtcGetErrorString(r) + "\n" + log);
  }
  size_t n = 0;
  r = nvrtcGetCUBINSize(prog, &n);
  if (r != NVRTC_SUCCESS || n == 0) {
    nvrtcDestroyProgram(&prog);
    return fail(FA_ECOMPILE, "nvrtcGetCUBINSize failed");
  }
  cubin.resize(n);
  nvrtcGetCUBIN(prog, &cubin[0]);
  nvrtcDestroyProgram(&prog);
  g_compile_count++;
  return FA_OK;
}

struct Kernel {
  std::string cubin;
  std::string entry;
  cudaLibrary_t lib = nullptr;
  cudaKernel_t fn = nullptr;
  int smem = 0;
  unsigned long long smem_set_mask = 0;  // devices on which the dynamic smem limit was raised
  fa_module* owner = nullptr;
  // device address of the kernel image's `fa_mod_buf` table per device (null: the image has none)
  void* buf_table[64] = {nullptr};
  unsigned long long buf_table_known = 0;
};

}  // namespace

constexpr int kMaxModBuffers = 8;

struct fa_module {
  std::string mod_source;
  std::map<std::string, Kernel*> kernels;  // key: template + defines
  const void* bufs[kMaxModBuffers] = {nullptr};  // device addresses of the captured buffers of the mods
  int nbufs = 0;
};

namespace {

const char* const kDefaultMods =
    "#define FA_HAS_SCORE_MOD 0\n#define FA_HAS_MASK_MOD 0\n"
    "__device__ __forceinline__ float fa_score_mod(float s, int, int, int, int) { return s; }\n"
    "__device__ __forceinline__ float fa_score_mod_grad(float, int, int, int, int) { return 1.0f; }\n"
    "__device__ __forceinline__ bool fa_mask_mod(int, int, int, int) { return true; }\n";

// Returns the compiled kernel `entry` of `tmpl` with the given defines (compiling if needed).
int get_kernel(fa_module* m, const std::string& tmpl, const std::string& defines, const std::string& entry,
               int smem, Kernel** out) {
  std::lock_guard<std::mutex> lk(g_mu);
  const std::string key = tmpl + "|" + defines + "|" + entry;
  auto it = m->kernels.find(key);
  if (it != m->kernels.end()) {
    *out = it->second;
    return FA_OK;
  }
  std::string th;
  if (int rc = templates_hash(th)) return rc;
  std::string src = defines + "\n" + m->mod_source + "\n#include \"" + tmpl + "\"\n";
  std::vector<std::string> opts = {"--gpu-architecture=sm_100a", "-std=c++17", "-lineinfo",
                                   "-I" + kernel_dir()};
  int major = 0, minor = 0;
  nvrtcVersion(&major, &minor);
  std::string h = hash_hex(src + "|" + th + "|" + std::to_string(major) + "." + std::to_string(minor));
  std::string cubin;
  const std::string cdir = cache_dir();
  const std::string cpath = cdir + "/" + h + ".cubin";
  bool from_cache = !cdir.empty() && read_file(cpath, cubin) && cubin.size() > 64;
  if (!from_cache) {
    if (int rc = nvrtc_compile(src, opts, cubin)) return rc;
    if (!cdir.empty()) {
      mkdirs(cdir);
      const std::string tmp = cpath + ".tmp" + std::to_string((long)getpid());
      std::ofstream f(tmp, std::ios::binary);
      if (f) {
        f.write(cubin.data(), (std::streamsize)cubin.size());
        f.close();
        rename(tmp.c_str(), cpath.c_str());
      }
    }
  }
  Kernel* k = new Kernel();
  k->cubin.swap(cubin);
  k->entry = entry;
  k->smem = smem;
  k->owner = m;
  m->kernels[key] = k;
  *out = k;
  return FA_OK;
}

// Loads the kernel on first launch and raises its dynamic shared-memory limit on this device.
int ready_kernel(Kernel* k) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (k->fn == nullptr) {
    FA_CUDA_CHECK(cudaLibraryLoadData(&k->lib, k->cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
    FA_CUDA_CHECK(cudaLibraryGetKernel(&k->fn, k->lib, k->entry.c_str()));
  }
  int dev = 0;
  FA_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 64 && !(k->smem_set_mask >> dev & 1ull)) {
    if (k->smem > 48 * 1024)
      FA_CUDA_CHECK(cudaFuncSetAttribute((const void*)k->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, k->smem));
    k->smem_set_mask |= 1ull << dev;
  }
  return FA_OK;
}

// Mods that read captured buffers find their addresses in the `fa_mod_buf` table of the kernel
// image: it is rewritten, in stream order, before every launch of a kernel of such a module.
int upload_buffers(Kernel* k, void* stream) {
  fa_module* m = k->owner;
  if (m == nullptr) return FA_OK;
  const void* local[kMaxModBuffers];
  int n = 0;
  void* table = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    n = m->nbufs;
    if (n == 0) return FA_OK;
    for (int i = 0; i < n; ++i) local[i] = m->bufs[i];
    int dev = 0;
    FA_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(FA_EUNSUPPORTED, "device ordinal above 63");
    if (!(k->buf_table_known >> dev & 1ull)) {
      void* dptr = nullptr;
      size_t bytes = 0;
      if (cudaLibraryGetGlobal(&dptr, &bytes, k->lib, "fa_mod_buf") != cudaSuccess) {
        cudaGetLastError();  // this kernel image does not reference the table
        dptr = nullptr;
      } else if (bytes < (size_t)n * sizeof(void*)) {
        return fail(FA_EINVAL, "fa_module_set_buffers: more buffers than the mod source declares");
      }
      k->buf_table[dev] = dptr;
      k->buf_table_known |= 1ull << dev;
    }
    table = k->buf_table[dev];
  }
  if (table != nullptr)
    FA_CUDA_CHECK(cudaMemcpyAsync(table, local, (size_t)n * sizeof(void*), cudaMemcpyHostToDevice, (cudaStream_t)stream));
  return FA_OK;
}

// ---- per-kernel device times (fa_profile_enable / fa_profile_read) -----------------------
// While profiling is on, every kernel launched by an entry point is bracketed by two CUDA events
// on the caller's stream.  The records belong to the calling thread and are reset at the start of
// each fa_fwd / fa_bwd / fa_decode call; the results of the call are the same with and without.
struct ProfRecord {
  const char* name;
  cudaEvent_t e0, e1;
};
std::atomic<int> g_profile_on{0};
thread_local std::vector<ProfRecord> t_prof;        // records of the most recent call
thread_local std::vector<cudaEvent_t> t_prof_pool;  // events of this thread, reused between calls
thread_local size_t t_prof_used = 0;
thread_local int t_prof_dev = -1;

void prof_reset() {
  if (!g_profile_on.load(std::memory_order_relaxed)) return;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return;
  if (dev != t_prof_dev) {  // events belong to the device that was current when they were made
    for (cudaEvent_t e : t_prof_pool) cudaEventDestroy(e);
    t_prof_pool.clear();
    t_prof_dev = dev;
  }
  t_prof.clear();
  t_prof_used = 0;
}
cudaEvent_t prof_event() {
  if (t_prof_used == t_prof_pool.size()) {
    cudaEvent_t e = nullptr;
    if (cudaEventCreate(&e) != cudaSuccess) return nullptr;
    t_prof_pool.push_back(e);
  }
  return t_prof_pool[t_prof_used++];
}
struct ProfScope {
  cudaStream_t st;
  cudaEvent_t e1 = nullptr;
  ProfScope(const char* name, void* stream) : st((cudaStream_t)stream) {
    if (!g_profile_on.load(std::memory_order_relaxed)) return;
    cudaEvent_t e0 = prof_event();
    e1 = prof_event();
    if (e0 == nullptr || e1 == nullptr) {
      e1 = nullptr;
      return;
    }
    cudaEventRecord(e0, st);
    t_prof.push_back({name, e0, e1});
  }
  ~ProfScope() {
    if (e1 != nullptr) cudaEventRecord(e1, st);
  }
};

int launch(Kernel* k, dim3 grid, dim3 block, void* params, void* stream) {
  if (int rc = ready_kernel(k)) return rc;
  if (int rc = upload_buffers(k, stream)) return rc;
  void* args[] = {params};
  ProfScope prof(k->entry.c_str(), stream);
  FA_CUDA_CHECK(cudaLaunchKernel((const void*)k->fn, grid, block, args, (size_t)k->smem, (cudaStream_t)stream));
  return FA_OK;
}

// ---- configuration ---------------------------------------------------------------------
int esize(int dtype) { return dtype == FA_F32 ? 4 : 2; }
int pitch(int cols, int es) { return cols * es + 16; }
constexpr int kMaxSmem = 227 * 1024;

struct FwdCfg {
  int BM, BN, warps, smem;
};
int fwd_smem(int dtype, int D, int Dv, int BM, int BN) {
  const int es = esize(dtype);
  int s = BM * pitch(D, es) + 2 * BN * pitch(D, es) + 2 * BN * pitch(Dv, es);
  if (dtype == FA_F32) s += BM * pitch(BN, 4);
  return s;
}
bool divides_or_single(int tile, int block, int nblocks) { return nblocks <= 1 || block % tile == 0; }

int pick_fwd(int dtype, int D, int Dv, int Sq, const FaTables* t, FwdCfg& c) {
  struct Cand { int BM, BN, warps; };
  std::vector<Cand> cands;
  if (dtype == FA_F32) {
    cands = {{64, 64, 4}, {64, 32, 4}, {32, 32, 2}, {16, 32, 1}, {16, 16, 1}};
  } else {
    if (D <= 64 && Sq > 64) cands.push_back({128, 64, 4});
    if (D <= 128 && Sq > 64) cands.push_back({128, 64, 8});
    cands.push_back({64, 64, 4});
    cands.push_back({64, 32, 4});
    cands.push_back({32, 32, 2});
    cands.push_back({16, 32, 1});
    cands.push_back({16, 16, 1});
  }
  for (auto& x : cands) {
    if (t && t->kv_num) {
      if (!divides_or_single(x.BM, t->QB, t->nQ) || !divides_or_single(x.BN, t->KVB, t->nKV)) continue;
    }
    const int s = fwd_smem(dtype, D, Dv, x.BM, x.BN);
    if (s > kMaxSmem) continue;
    c = {x.BM, x.BN, x.warps, s};
    return FA_OK;
  }
  return fail(FA_EUNSUPPORTED, "no forward tile configuration fits this head dim / BlockMask block size "
                               "(block sizes must be multiples of 16 unless there is a single block)");
}

struct BwdCfg {
  int tile, warps, smem_dq, smem_dkdv;
};
int pick_bwd(int dtype, int D, int Dv, const FaTables* t, BwdCfg& c) {
  const int es = esize(dtype);
  for (int warps : {4, 2, 1}) {
    const int T = 16 * warps;
    if (t && t->kv_num) {
      if (!divides_or_single(T, t->QB, t->nQ) || !divides_or_single(T, t->KVB, t->nKV)) continue;
    }
    const int pq = pitch(D, es), pv = pitch(Dv, es);
    const int f32x = dtype == FA_F32 ? T * pitch(T, 4) : 0;
    const int dq = T * pq + T * pv + 2 * T * pq + 2 * T * pv + f32x;
    const int dkdv = T * pq + T * pv + 2 * T * pq + 2 * T * pv + 2 * (2 * T * 4) + f32x;
    if (dq > kMaxSmem || dkdv > kMaxSmem) continue;
    c = {T, warps, dq, dkdv};
    return FA_OK;
  }
  return fail(FA_EUNSUPPORTED, "no backward tile configuration fits this head dim / BlockMask block size");
}

struct DecCfg {
  int BM, BN, stages, smem;
};
int pick_decode(int dtype, int D, int Dv, int Sq, const FaTables* t, DecCfg& c) {
  if (dtype == FA_F32) return fail(FA_EUNSUPPORTED, "the decode kernel takes fp16 / bf16 inputs");
  if (Sq > 64) return fail(FA_EUNSUPPORTED, "the decode kernel handles at most 64 query rows");
  if (t && t->kv_num && t->nQ != 1) return fail(FA_EUNSUPPORTED, "decode needs a BlockMask with a single q block");
  const int BM = Sq <= 16 ? 16 : (Sq <= 32 ? 32 : 64);
  const int CG = 4 / (BM / 16);
  for (int BN : {128, 64, 32, 16}) {
    if (BN / CG < 16) continue;
    if (D > 64 && BN > 64) continue;
    if (t && t->kv_num && !divides_or_single(BN, t->KVB, t->nKV)) continue;
    // Two stages first: the kernel is bound by the latency its few resident warps can hide, and
    // the smaller ring lets a third CTA share the SM (B32 H8 Skv16384 D64: 0.187 ms with two
    // stages against 0.218 ms with three at one query row, 0.224 against 0.269 at sixteen).
    for (int stages : {2, 3}) {
      const int pipe = stages * (BN * pitch(D, 2) + BN * pitch(Dv, 2));
      const int mrg = CG * BM * (Dv + 4) * 4;
      const int smem = BM * pitch(D, 2) + (pipe > mrg ? pipe : mrg);
      if (smem > kMaxSmem) continue;
      c = {BM, BN, stages, smem};
      return FA_OK;
    }
  }
  return fail(FA_EUNSUPPORTED, "no decode tile configuration fits this head dim / BlockMask block size");
}

std::string defs(std::initializer_list<std::pair<const char*, int>> kv) {
  std::string s;
  for (auto& p : kv) s += std::string("#define ") + p.first + " " + std::to_string(p.second) + "\n";
  return s;
}

// ---- argument validation ---------------------------------------------------------------
int check_tensor(const fa_tensor& t, const char* name, int es, bool required = true) {
  if (t.ptr == nullptr) return required ? fail(FA_EINVAL, std::string(name) + ": null pointer") : FA_OK;
  if (((uintptr_t)t.ptr & 15) != 0) return fail(FA_EINVAL, std::string(name) + ": pointer must be 16-byte aligned");
  if ((t.stride_b * es) % 16 || (t.stride_h * es) % 16 || (t.stride_s * es) % 16)
    return fail(FA_EINVAL, std::string(name) + ": byte strides must be multiples of 16");
  return FA_OK;
}
FaTensor cvt(const fa_tensor& t) { return FaTensor{t.ptr, t.stride_b, t.stride_h, t.stride_s}; }

int check_common(fa_module* m, const fa_attn_params* p) {
  if (!m) return fail(FA_EINVAL, "module is null");
  if (!p) return fail(FA_EINVAL, "params is null");
  if (p->dtype < FA_F16 || p->dtype > FA_F32) return fail(FA_EINVAL, "unknown dtype");
  if (p->B <= 0 || p->Hq <= 0 || p->Hkv <= 0 || p->Sq <= 0 || p->Skv <= 0)
    return fail(FA_EINVAL, "B, Hq, Hkv, Sq, Skv must be positive");
  if (p->Hq % p->Hkv) return fail(FA_EINVAL, "Hq must be a multiple of Hkv");
  if (p->D <= 0 || p->D % 16 || p->Dv <= 0 || p->Dv % 16)
    return fail(FA_EUNSUPPORTED, "head dims must be positive multiples of 16");
  if (p->Dv > p->D) return fail(FA_EINVAL, "value head dim must not exceed the query/key head dim");
  if (p->D > 256) return fail(FA_EUNSUPPORTED, "head dim above 256 is not supported");
  if (p->B > 65535 || p->Hq > 65535) return fail(FA_EUNSUPPORTED, "B and Hq must not exceed 65535");
  const int es = esize(p->dtype);
  if (int rc = check_tensor(p->q, "q", es)) return rc;
  if (int rc = check_tensor(p->k, "k", es)) return rc;
  if (int rc = check_tensor(p->v, "v", es)) return rc;
  if (int rc = check_tensor(p->o, "o", es)) return rc;
  const fa_block_tables& t = p->tables;
  if (t.kv_num_blocks) {
    if (!t.kv_indices) return fail(FA_EINVAL, "kv_indices is null");
    if ((t.full_kv_num_blocks == nullptr) != (t.full_kv_indices == nullptr))
      return fail(FA_EINVAL, "full_kv_num_blocks and full_kv_indices must be both given or both null");
    if (t.num_q_blocks <= 0 || t.num_kv_blocks <= 0 || t.q_block_size <= 0 || t.kv_block_size <= 0)
      return fail(FA_EINVAL, "BlockMask grid and block sizes must be positive");
    if (!(t.mask_B == 1 || t.mask_B == p->B) || !(t.mask_H == 1 || t.mask_H == p->Hq))
      return fail(FA_EINVAL, "BlockMask batch/head dims must be 1 or match B/Hq");
    if ((long long)t.num_q_blocks * t.q_block_size < p->Sq || (long long)t.num_kv_blocks * t.kv_block_size < p->Skv)
      return fail(FA_EINVAL, "BlockMask does not cover the sequence lengths");
  }
  if (t.mask_bits) {
    if (!t.kv_num_blocks) return fail(FA_EINVAL, "mask_bits come with the BlockMask tables they were built beside");
    if (((uintptr_t)t.mask_bits & 15) || t.mask_bits_stride % 4 || t.mask_bits_stride * 32 < p->Skv || t.mask_bits_rows < p->Sq)
      return fail(FA_EINVAL, "mask_bits: 16-byte aligned, rows of a multiple of 4 words that cover Skv, at least Sq rows");
    if (!(t.mask_bits_B == 1 || t.mask_bits_B == p->B) || !(t.mask_bits_H == 1 || t.mask_bits_H == p->Hq))
      return fail(FA_EINVAL, "mask_bits batch/head dims must be 1 or match B/Hq");
  }
  return FA_OK;
}

FaTables cvt_tables(const fa_block_tables& t) {
  FaTables r;
  r.kv_num = t.kv_num_blocks; r.kv_idx = t.kv_indices;
  r.full_kv_num = t.full_kv_num_blocks; r.full_kv_idx = t.full_kv_indices;
  r.q_num = t.q_num_blocks; r.q_idx = t.q_indices;
  r.full_q_num = t.full_q_num_blocks; r.full_q_idx = t.full_q_indices;
  r.mB = t.mask_B; r.mH = t.mask_H; r.nQ = t.num_q_blocks; r.nKV = t.num_kv_blocks;
  r.QB = t.q_block_size; r.KVB = t.kv_block_size;
  r.mask_bits = t.mask_bits; r.mask_stride = t.mask_bits_stride; r.mask_rows = t.mask_bits_rows;
  r.mask_B = t.mask_bits_B; r.mask_H = t.mask_bits_H;
  return r;
}

void fill_params(const fa_attn_params* p, FaParams& k) {
  memset(&k, 0, sizeof k);
  k.q = cvt(p->q); k.k = cvt(p->k); k.v = cvt(p->v); k.o = cvt(p->o);
  k.lse = p->lse; k.status = p->status;
  k.B = p->B; k.Hq = p->Hq; k.Hkv = p->Hkv; k.Sq = p->Sq; k.Skv = p->Skv; k.D = p->D; k.Dv = p->Dv;
  k.b_off = p->b_offset; k.h_off = p->h_offset; k.scale = p->scale;
  k.t = cvt_tables(p->tables);
}

// ---- kernels that do not depend on the mods --------------------------------------------

// One warp per table row.  The reference orders a row by a stable descending argsort of the
// 0/1 block grid (flaxattention/core/blockmask.py:57-64): set columns ascending, then the
// unset columns ascending.  `transposed` builds the q-tables from the same class grid.
__global__ void fa_tables_kernel(const signed char* __restrict__ cls, int rows_per_bh, int cols, int want,
                                 bool transposed, int nQ, int nKV, long long n_rows,
                                 int* __restrict__ num_out, int* __restrict__ idx_out) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int lane = threadIdx.x & 31;
  const long long bh = row / rows_per_bh;
  const int r = (int)(row - bh * rows_per_bh);
  const signed char* g = cls + bh * (long long)nQ * nKV;
  auto is_set = [&](int c) -> bool {
    const signed char v = transposed ? g[(long long)c * nKV + r] : g[(long long)r * nKV + c];
    return v == want;
  };
  int total = 0;
  for (int c0 = 0; c0 < cols; c0 += 32) {
    const int c = c0 + lane;
    const bool s = c < cols && is_set(c);
    total += __popc(__ballot_sync(0xffffffffu, s));
  }
  int n_set = 0, n_unset = 0;
  int* out = idx_out + row * cols;
  for (int c0 = 0; c0 < cols; c0 += 32) {
    const int c = c0 + lane;
    const bool in = c < cols;
    const bool s = in && is_set(c);
    const unsigned bs = __ballot_sync(0xffffffffu, s);
    const unsigned bu = __ballot_sync(0xffffffffu, in && !s);
    const unsigned lt = (1u << lane) - 1u;
    if (s) out[n_set + __popc(bs & lt)] = c;
    else if (in) out[total + n_unset + __popc(bu & lt)] = c;
    n_set += __popc(bs);
    n_unset += __popc(bu);
  }
  if (lane == 0) num_out[row] = total;
}


// delta[b,h,q] = sum_d O[b,h,q,d] * dO[b,h,q,d]  (flaxattention/kernel/attention.py:338-345).
// LPR lanes cooperate on one row; each lane reads 16-byte pieces.
template <int DT, int LPR>
__global__ void fa_delta_kernel(FaTensor o, FaTensor dout, float* __restrict__ delta, int Hq, int Sq, int Dv,
                                long long n_rows) {
  constexpr int ES = DT == FA_F32 ? 4 : 2;
  constexpr int EPC = 16 / ES;  // elements per 16-byte chunk
  const long long gt = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = gt / LPR;
  const int sub = (int)(gt % LPR);
  float acc = 0.f;
  if (row < n_rows) {
    const long long bh = row / Sq;
    const int q = (int)(row - bh * Sq);
    const int b = (int)(bh / Hq), h = (int)(bh - (long long)b * Hq);
    const char* po = (const char*)o.ptr + ((long long)b * o.sb + (long long)h * o.sh + (long long)q * o.ss) * ES;
    const char* pd = (const char*)dout.ptr + ((long long)b * dout.sb + (long long)h * dout.sh + (long long)q * dout.ss) * ES;
    for (int c = sub; c * EPC < Dv; c += LPR) {
      const uint4 a = *(const uint4*)(po + c * 16);
      const uint4 d = *(const uint4*)(pd + c * 16);
      const unsigned aw[4] = {a.x, a.y, a.z, a.w}, dw[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (DT == FA_F32) {
          acc += __uint_as_float(aw[i]) * __uint_as_float(dw[i]);
        } else if (DT == FA_F16) {
          const __half2 ha = *reinterpret_cast<const __half2*>(&aw[i]);
          const __half2 hd = *reinterpret_cast<const __half2*>(&dw[i]);
          const float2 fa = __half22float2(ha), fd = __half22float2(hd);
          acc += fa.x * fd.x + fa.y * fd.y;
        } else {
          acc += __uint_as_float(aw[i] << 16) * __uint_as_float(dw[i] << 16) +
                 __uint_as_float(aw[i] & 0xffff0000u) * __uint_as_float(dw[i] & 0xffff0000u);
        }
      }
    }
  }
#pragma unroll
  for (int off = LPR / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (row < n_rows && sub == 0) delta[row] = acc;
}

// Per-row scalars of the tcgen05 backward, padded to whole 128-row tiles so that a q tile's
// values are one aligned 512-byte run: nlse2 = -lse * log2(e) (-inf for rows without mass or
// beyond Sq, which makes p = 0 there) and ndelta = -sum_d O * dO (0 beyond Sq).
// The same pass zeroes the dQ accumulation buffer when `dq_acc` is given (D floats per padded
// row, whatever their order inside a tile): one launch and one pass less than a separate memset.
template <int DT, int LPR>
__global__ void fa_bwd_prep_kernel(FaTensor o, FaTensor dout, const float* __restrict__ lse, float* __restrict__ nlse2,
                                   float* __restrict__ ndelta, float* __restrict__ dq_acc, int* __restrict__ work_counter,
                                   int Hq, int Sq, int sq_pad, int Dv, int D, int n_bh) {
  // grid: x over groups of R * (256 / LPR) padded rows of one (batch, head), LPR lanes per row; (y, z) over the heads.
  // A thread works on R rows, 256 / LPR apart, and has the loads of all of them in flight before it uses the first
  // (Dv <= 128: at most two 16-byte pieces of O and of dO per lane and row).
  constexpr int R = 4, ROWS = 256 / LPR;
  const int bh = blockIdx.y + blockIdx.z * gridDim.y;
  const int rloc = threadIdx.x / LPR, sub = threadIdx.x % LPR;
  const int q0 = blockIdx.x * (R * ROWS) + rloc;
  if (work_counter != nullptr && blockIdx.x == 0 && threadIdx.x == 0 && bh == 0) *work_counter = 0;  // the item counter of the backward kernel
  if (bh >= n_bh) return;
  const int b = bh / Hq, h = bh - b * Hq;
  const int nc = Dv / 8;  // 16-byte pieces per row
  uint4 a[R][2], d[R][2];
  float l[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int q = q0 + r * ROWS;
    const bool valid = q < Sq;
    const char* po = (const char*)o.ptr + ((long long)b * o.sb + (long long)h * o.sh + (long long)q * o.ss) * 2;
    const char* pd = (const char*)dout.ptr + ((long long)b * dout.sb + (long long)h * dout.sh + (long long)q * dout.ss) * 2;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int c = sub + k * LPR;
      const bool have = valid && c < nc;
      a[r][k] = have ? *(const uint4*)(po + c * 16) : make_uint4(0u, 0u, 0u, 0u);
      d[r][k] = have ? *(const uint4*)(pd + c * 16) : make_uint4(0u, 0u, 0u, 0u);
    }
    l[r] = (valid && sub == 0) ? lse[(long long)bh * Sq + q] : 0.f;
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int q = q0 + r * ROWS;
    if (q >= sq_pad) continue;  // (whole lanes groups of a row leave together)
    const long long row = (long long)bh * sq_pad + q;
    if (dq_acc != nullptr) {
      float4* z = (float4*)(dq_acc + row * D);
      for (int i = sub; i < D / 4; i += LPR) z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const unsigned aw[4] = {a[r][k].x, a[r][k].y, a[r][k].z, a[r][k].w}, dw[4] = {d[r][k].x, d[r][k].y, d[r][k].z, d[r][k].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (DT == FA_F16) {
          const float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&aw[i]));
          const float2 fd = __half22float2(*reinterpret_cast<const __half2*>(&dw[i]));
          acc += fa.x * fd.x + fa.y * fd.y;
        } else {
          acc += __uint_as_float(aw[i] << 16) * __uint_as_float(dw[i] << 16) +
                 __uint_as_float(aw[i] & 0xffff0000u) * __uint_as_float(dw[i] & 0xffff0000u);
        }
      }
    }
#pragma unroll
    for (int off = LPR / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (sub == 0) {
      const bool valid = q < Sq;
      nlse2[row] = (valid && l[r] != -INFINITY) ? -l[r] * 1.4426950408889634f : -INFINITY;
      ndelta[row] = valid ? -acc : 0.f;
    }
  }
}

// dq = scale * dq_acc for the tcgen05 backward.  The fp32 accumulation buffer holds, per
// (b, h, 128-row q tile), two [128 rows][32 columns] blocks (columns 0-31, then 32-63), and the
// eight 16-byte chunks of a block row r sit at position k ^ (r & 7).
template <int DT>
__global__ void fa_dq_convert_kernel(const float* __restrict__ acc, FaTensor dq, int Hq, int Sq, int sq_pad, float scale,
                                     int n_bh) {
  // grid: x over the rows of one (batch, head), one 8-element output chunk per thread; (y, z) over the heads
  const int bh = blockIdx.y + blockIdx.z * gridDim.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int k8 = i & 7, q = i >> 3;
  if (bh >= n_bh || q >= Sq) return;
  const int b = bh / Hq, h = bh - b * Hq;
  const int r = q & 127, c = 2 * (k8 & 3);
  const float* src = acc + ((long long)bh * sq_pad + (q - r)) * 64 + (k8 >> 2) * (128 * 32) + r * 32;
  const float4 lo = *(const float4*)(src + ((c ^ (r & 7)) * 4));
  const float4 hi = *(const float4*)(src + (((c + 1) ^ (r & 7)) * 4));
  char* dst = (char*)dq.ptr + ((long long)b * dq.sb + (long long)h * dq.sh + (long long)q * dq.ss) * 2 + k8 * 16;
  if (DT == FA_F16) {
    __half2 o[4] = {__floats2half2_rn(lo.x * scale, lo.y * scale), __floats2half2_rn(lo.z * scale, lo.w * scale),
                    __floats2half2_rn(hi.x * scale, hi.y * scale), __floats2half2_rn(hi.z * scale, hi.w * scale)};
    *(uint4*)dst = *reinterpret_cast<uint4*>(o);
  } else {
    __nv_bfloat162 o[4] = {__floats2bfloat162_rn(lo.x * scale, lo.y * scale), __floats2bfloat162_rn(lo.z * scale, lo.w * scale),
                           __floats2bfloat162_rn(hi.x * scale, hi.y * scale), __floats2bfloat162_rn(hi.z * scale, hi.w * scale)};
    *(uint4*)dst = *reinterpret_cast<uint4*>(o);
  }
}

// The same for head dim 128, where the kernel accumulates dQ transposed: per (b, h, 64-row q
// tile) the buffer holds two [128 head-dim lanes][32 query columns] blocks (query columns 0-31,
// then 32-63), 16-byte chunks of a block row d at position k ^ (d & 7).  A warp takes 32
// consecutive query rows and one group of 8 head-dim values: each of its 8 reads is one 128-byte
// row of a block, and every thread writes one 16-byte chunk of its output row.
template <int DT>
__global__ void fa_dq_convert_t_kernel(const float* __restrict__ acc, FaTensor dq, int Hq, int Sq, int sq_pad, float scale,
                                       int n_bh) {
  const int bh = blockIdx.y + blockIdx.z * gridDim.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int dg = (i >> 5) & 15, q = ((i >> 9) << 5) | (i & 31);
  if (bh >= n_bh || q >= Sq) return;
  const int b = bh / Hq, h = bh - b * Hq;
  const int c = q & 63, hf = c >> 5, k = (c & 31) >> 2, w = c & 3;
  const float* src = acc + ((long long)bh * (sq_pad >> 6) + (q >> 6)) * (128 * 64) + hf * (128 * 32) + w;
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int d = dg * 8 + j;
    v[j] = src[d * 32 + ((k ^ (d & 7)) << 2)] * scale;
  }
  char* dst = (char*)dq.ptr + ((long long)b * dq.sb + (long long)h * dq.sh + (long long)q * dq.ss) * 2 + dg * 16;
  if (DT == FA_F16) {
    __half2 o[4] = {__floats2half2_rn(v[0], v[1]), __floats2half2_rn(v[2], v[3]), __floats2half2_rn(v[4], v[5]),
                    __floats2half2_rn(v[6], v[7])};
    *(uint4*)dst = *reinterpret_cast<uint4*>(o);
  } else {
    __nv_bfloat162 o[4] = {__floats2bfloat162_rn(v[0], v[1]), __floats2bfloat162_rn(v[2], v[3]),
                           __floats2bfloat162_rn(v[4], v[5]), __floats2bfloat162_rn(v[6], v[7])};
    *(uint4*)dst = *reinterpret_cast<uint4*>(o);
  }
}

// Combines the per-split partial results of the decode kernels: one warp per output row.  Lane s
// takes the (max, sum) pair of split s and its weight 2^(m_s - m*), 32 splits at a time; the
// weights then go round by shuffle while every lane accumulates its output columns, each read of
// a partial row being one contiguous run of floats.
template <int DT>
__global__ void fa_decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         FaTensor o, float* __restrict__ lse, int Hq, int Sq, int Dv, int ns,
                                         long long n_rows) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int lane = threadIdx.x & 31;
  const long long bh = row / Sq;
  const int q = (int)(row - bh * Sq);
  const int b = (int)(bh / Hq), h = (int)(bh - (long long)b * Hq);
  auto prow = [&](int s) -> long long { return (bh * ns + s) * Sq + q; };
  float mstar = -INFINITY;
  for (int s0 = 0; s0 < ns; s0 += 32)
    if (s0 + lane < ns) mstar = fmaxf(mstar, part_ml[prow(s0 + lane) * 2]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mstar = fmaxf(mstar, __shfl_xor_sync(0xffffffffu, mstar, off));
  constexpr int MAXC = 8;  // output columns per lane: head dims up to 256
  float acc[MAXC];
#pragma unroll
  for (int c = 0; c < MAXC; ++c) acc[c] = 0.f;
  float lstar = 0.f;
  for (int s0 = 0; s0 < ns; s0 += 32) {
    float w = 0.f;
    if (s0 + lane < ns) {
      const float2 ml = *(const float2*)(part_ml + prow(s0 + lane) * 2);
      w = ml.x == -INFINITY ? 0.f : exp2f(ml.x - mstar);
      lstar += w * ml.y;
    }
    const int cnt = ns - s0 < 32 ? ns - s0 : 32;
    for (int t = 0; t < cnt; ++t) {
      const float wt = __shfl_sync(0xffffffffu, w, t);
      if (wt == 0.f) continue;
      const float* src = part_o + prow(s0 + t) * Dv;
#pragma unroll
      for (int c = 0; c < MAXC; ++c)
        if (c * 32 + lane < Dv) acc[c] += wt * src[c * 32 + lane];
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) lstar += __shfl_xor_sync(0xffffffffu, lstar, off);
  const float inv = lstar > 0.f ? 1.f / lstar : 0.f;
  char* og = (char*)o.ptr + ((long long)b * o.sb + (long long)h * o.sh + (long long)q * o.ss) * 2;
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int col = c * 32 + lane;
    if (col < Dv) {
      if (DT == FA_F16) ((__half*)og)[col] = __float2half_rn(acc[c] * inv);
      else ((__nv_bfloat16*)og)[col] = __float2bfloat16_rn(acc[c] * inv);
    }
  }
  if (lane == 0 && lse != nullptr) lse[row] = lstar > 0.f ? (mstar + log2f(lstar)) * 0.6931471805599453f : -INFINITY;
}

}  // namespace

// ======================================================================================
// C ABI
// ======================================================================================
extern "C" {

const char* fa_last_error(void) { return g_err.c_str(); }
int fa_version(void) { return 100; }

int fa_set_kernel_dir(const char* path) {
  if (!path) return fail(FA_EINVAL, "path is null");
  std::lock_guard<std::mutex> lk(g_mu);
  g_kernel_dir = path;
  g_templates_hash.clear();
  return FA_OK;
}
int fa_set_cache_dir(const char* path) {
  if (!path) return fail(FA_EINVAL, "path is null");
  std::lock_guard<std::mutex> lk(g_mu);
  g_cache_dir = path;
  g_cache_dir_set = true;
  return FA_OK;
}
int fa_compile_count(void) { return g_compile_count.load(); }

int fa_profile_enable(int on) {
  g_profile_on.store(on ? 1 : 0);
  return FA_OK;
}
int fa_profile_read(int max_kernels, float* ms, const char** names) {
  const int n = (int)t_prof.size();
  if (n == 0) return 0;
  if (max_kernels > 0 && (!ms || !names)) return fail(FA_EINVAL, "ms and names are required");
  FA_CUDA_CHECK(cudaEventSynchronize(t_prof.back().e1));
  for (int i = 0; i < n && i < max_kernels; ++i) {
    FA_CUDA_CHECK(cudaEventElapsedTime(&ms[i], t_prof[i].e0, t_prof[i].e1));
    names[i] = t_prof[i].name;
  }
  return n;
}

int fa_selftest_bounded_wait(unsigned long long limit_ns, int* status, int* gave_up, unsigned long long* waited_ns,
                             void* stream) {
  if (!status || !gave_up || !waited_ns) return fail(FA_EINVAL, "status, gave_up and waited_ns are required");
  if (limit_ns < 1000ull || limit_ns > 100000000ull) return fail(FA_EINVAL, "limit between 1 us and 100 ms");
  static fa_module* mod = nullptr;  // owns the compiled self-test kernels (one per limit)
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!mod) {
      mod = new fa_module();
      mod->mod_source = kDefaultMods;
    }
  }
  Kernel* k = nullptr;
  const std::string defs = "#define FA_WAIT_LIMIT_NS " + std::to_string(limit_ns) + "ull\n";
  if (int rc = get_kernel(mod, "fa_selftest.cuh", defs, "fa_wait_selftest_kernel", 0, &k)) return rc;
  struct { int* status; int* gave_up; unsigned long long* waited_ns; } prm = {status, gave_up, waited_ns};
  return launch(k, dim3(1), dim3(64), &prm, stream);
}

int fa_module_create(const char* mod_source, fa_module** out) {
  if (!out) return fail(FA_EINVAL, "out is null");
  fa_module* m = new fa_module();
  m->mod_source = (mod_source && *mod_source) ? mod_source : kDefaultMods;
  *out = m;
  return FA_OK;
}

int fa_module_set_buffers(fa_module* m, const void* const* ptrs, int n) {
  if (!m) return fail(FA_EINVAL, "module is null");
  if (n < 0 || n > kMaxModBuffers) return fail(FA_EINVAL, "between 0 and 8 captured buffers");
  if (n > 0 && !ptrs) return fail(FA_EINVAL, "ptrs is null");
  for (int i = 0; i < n; ++i)
    if (!ptrs[i]) return fail(FA_EINVAL, "captured buffer " + std::to_string(i) + " is null");
  std::lock_guard<std::mutex> lk(g_mu);
  for (int i = 0; i < n; ++i) m->bufs[i] = ptrs[i];
  m->nbufs = n;
  return FA_OK;
}

void fa_module_destroy(fa_module* m) {
  if (!m) return;
  for (auto& kv : m->kernels) {
    if (kv.second->lib) cudaLibraryUnload(kv.second->lib);
    delete kv.second;
  }
  delete m;
}

}  // extern "C"

namespace {

int round_flag(int dtype, int flags) { return (dtype != FA_F32 && (flags & FA_FLAG_ROUND_SCORES)) ? 1 : 0; }

int get_fwd_kernel(fa_module* m, int dtype, int D, int Dv, int flags, const FwdCfg& c, Kernel** k) {
  return get_kernel(m, "fa_fwd.cuh",
                    defs({{"FA_DTYPE", dtype}, {"FA_D", D}, {"FA_DV", Dv}, {"FA_BM", c.BM}, {"FA_BN", c.BN},
                          {"FA_WARPS", c.warps}, {"FA_ROUND_SCORES", round_flag(dtype, flags)}}),
                    "fa_fwd_kernel", c.smem, k);
}
int get_bwd_kernel(fa_module* m, int dtype, int D, int Dv, int flags, const BwdCfg& c, bool dq, Kernel** k) {
  return get_kernel(m, "fa_bwd.cuh",
                    defs({{"FA_DTYPE", dtype}, {"FA_D", D}, {"FA_DV", Dv}, {"FA_BQ", c.tile}, {"FA_BK", c.tile},
                          {"FA_WARPS", c.warps}, {"FA_ROUND_SCORES", round_flag(dtype, flags)}}),
                    dq ? "fa_bwd_dq_kernel" : "fa_bwd_dkdv_kernel", dq ? c.smem_dq : c.smem_dkdv, k);
}
int get_decode_kernel(fa_module* m, int dtype, int D, int Dv, int flags, const DecCfg& c, bool pack, Kernel** k) {
  return get_kernel(m, "fa_decode.cuh",
                    defs({{"FA_DTYPE", dtype}, {"FA_D", D}, {"FA_DV", Dv}, {"FA_BM", c.BM}, {"FA_BN", c.BN},
                          {"FA_STAGES", c.stages}, {"FA_ROUND_SCORES", round_flag(dtype, flags)},
                          {"FA_PACK_HEADS", pack ? 1 : 0}}),
                    "fa_decode_kernel", c.smem, k);
}
// Grouped-query decode: the G query heads of a kv head share one CTA (their G * Sq rows form one
// tile and K / V are read once) when the rows fit a tile and the kv walk is the same for every
// head of the group, i.e. there are no tables or the tables are broadcast over the heads.
bool decode_packs_heads(const fa_attn_params* p) {
  if (p->Hkv <= 0 || p->Hq % p->Hkv) return false;
  const int G = p->Hq / p->Hkv;
  if (G <= 1 || p->dtype == FA_F32 || (long long)G * p->Sq > 64) return false;
  return p->tables.kv_num_blocks == nullptr || p->tables.mask_H == 1;
}
// ---- tcgen05 forward: TMA tensor maps and dispatch -----------------------------------------
struct alignas(64) FaTensorMapHost {
  unsigned long long v[16];
};
static_assert(sizeof(FaTensorMapHost) == sizeof(CUtensorMap), "tensor map size");
struct FaTcParamsHost {
  FaParams p;
  FaTensorMapHost tq, tk, tv, to;
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode_tiled = nullptr;

int encode_fn(EncodeTiledFn* out) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_encode_tiled) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    FA_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    if (!fn || q != cudaDriverEntryPointSuccess) return fail(FA_ECUDA, "cuTensorMapEncodeTiled is not available");
    g_encode_tiled = (EncodeTiledFn)fn;
  }
  *out = g_encode_tiled;
  return FA_OK;
}

// 4-d map (D, S, H, B) over a [.., S, D]-strided tensor; box = 64 elements x box_rows rows, 128-byte swizzle
int make_map(FaTensorMapHost* out, int dtype, const fa_tensor& t, int D, int S, int H, int B, int box_rows = 128) {
  EncodeTiledFn enc = nullptr;
  if (int rc = encode_fn(&enc)) return rc;
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  const cuuint64_t strides[3] = {(cuuint64_t)t.stride_s * 2, (cuuint64_t)t.stride_h * 2, (cuuint64_t)t.stride_b * 2};
  const cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc((CUtensorMap*)out, dtype == FA_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                   t.ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FA_ECUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return FA_OK;
}

// Shapes the tcgen05 forward kernel covers; everything else runs on the general kernel.
bool tc_fwd_eligible(const fa_attn_params* p) {
  if (p->flags & FA_FLAG_GENERAL_KERNELS) return false;
  if (p->dtype == FA_F32) return false;
  if (p->D != p->Dv || !(p->D == 64 || p->D == 128)) return false;
  if (p->Sq < 128 || p->Skv > 32768) return false;
  if (!(p->scale > 0.f)) return false;  // the kernel takes row maxima over unscaled scores
  const fa_block_tables& t = p->tables;
  if (t.kv_num_blocks) {
    if (!(t.num_q_blocks == 1 || t.q_block_size % 128 == 0)) return false;
    if (!(t.num_kv_blocks == 1 || t.kv_block_size % 128 == 0)) return false;
  }
  // byte strides above the row must stay below 2^40 (tensor-map limit); rows are 16-byte aligned already
  return true;
}

// decode = true selects the split-KV variant of the kernel (one query tile per CTA, partial results)
int get_fwd_tc_kernel(fa_module* m, int dtype, int D, int flags, Kernel** k, bool decode = false) {
  // must match the shared-memory map of fa_fwd_tc.cuh (fa_tc::SMEM_BYTES)
  const int atoms = D / 64, nstage = decode ? 5 : (D == 64 ? 3 : 2);
  const int smem = 2 * atoms * 16384 + 2 * nstage * atoms * 16384 + (1 + 4 * nstage + 8) * 8 + 16 + 256 * 2 + 256 * 2 +
                   2 * 256 + (256 / 32) * 4 + 1024;
  std::string d = defs({{"FA_DTYPE", dtype}, {"FA_D", D}, {"FA_ROUND_SCORES", round_flag(dtype, flags)}, {"FA_TC_DECODE", decode ? 1 : 0}});
  return get_kernel(m, "fa_fwd_tc.cuh", d, "fa_fwd_tc_kernel", smem, k);
}

// Shapes the split-KV variant of the tcgen05 kernel covers (`num_splits` CTAs per (batch, head), one
// partial result per CTA and row); everything else runs on the general decode kernel.
bool tc_decode_eligible(const fa_attn_params* p) {
  if (p->flags & FA_FLAG_GENERAL_KERNELS) return false;
  if (p->dtype == FA_F32) return false;
  if (p->D != 64 || p->Dv != 64) return false;
  // The kernel gives every query row two threads (64 kv columns of a tile each), whatever Sq is:
  // measured on B32 H8 Skv16384 against the general decode kernel it takes 0.225 ms at 64 rows
  // (general: 0.55), 0.209 at 16 (general: 0.231), 0.209 at 2 and 0.208 at 1 (general: 0.206): it
  // streams K / V through TMA and a five-stage ring at the same rate whatever the row count, so it
  // takes everything from two rows up.
  if (p->Sq < 2 || p->Sq > 64 || p->Skv < 1024 || p->Skv > 32768) return false;
  if (!(p->scale > 0.f)) return false;
  const fa_block_tables& t = p->tables;
  if (t.kv_num_blocks) {
    if (t.num_q_blocks != 1) return false;
    if (!(t.num_kv_blocks == 1 || t.kv_block_size % 128 == 0)) return false;
  }
  return true;
}
int launch_decode_tc(fa_module* m, const fa_attn_params* p, const FaParams& kp, int num_splits, void* stream) {
  Kernel* k = nullptr;
  if (int rc = get_fwd_tc_kernel(m, p->dtype, p->D, p->flags, &k, true)) return rc;
  FaTcParamsHost tp;
  tp.p = kp;
  if (int rc = make_map(&tp.tq, p->dtype, p->q, p->D, p->Sq, p->Hq, p->B, 64)) return rc;  // the queries go into a tile twice
  if (int rc = make_map(&tp.tk, p->dtype, p->k, p->D, p->Skv, p->Hkv, p->B)) return rc;
  if (int rc = make_map(&tp.tv, p->dtype, p->v, p->Dv, p->Skv, p->Hkv, p->B)) return rc;
  memset(&tp.to, 0, sizeof(tp.to));  // (the decode variant writes partial results, not the output)
  return launch(k, dim3(num_splits, p->Hq, p->B), dim3(384), &tp, stream);
}

int launch_fwd_tc(fa_module* m, const fa_attn_params* p, const FaParams& kp, void* stream) {
  Kernel* k = nullptr;
  if (int rc = get_fwd_tc_kernel(m, p->dtype, p->D, p->flags, &k)) return rc;
  FaTcParamsHost tp;
  tp.p = kp;
  if (int rc = make_map(&tp.tq, p->dtype, p->q, p->D, p->Sq, p->Hq, p->B)) return rc;
  if (int rc = make_map(&tp.tk, p->dtype, p->k, p->D, p->Skv, p->Hkv, p->B)) return rc;
  if (int rc = make_map(&tp.tv, p->dtype, p->v, p->Dv, p->Skv, p->Hkv, p->B)) return rc;
  if (int rc = make_map(&tp.to, p->dtype, p->o, p->Dv, p->Sq, p->Hq, p->B)) return rc;
  // Heads vary fastest and the query tile pair slowest (the kernel walks the pairs from the last one
  // down), so that under a causal mask the CTAs with the most kv tiles are dispatched first for
  // all heads: longest-first order keeps the tail of the grid short.
  return launch(k, dim3(p->Hq, p->B, (p->Sq + 255) / 256), dim3(384), &tp, stream);
}

// ---- tcgen05 backward ----------------------------------------------------------------------
struct FaBwdTcParamsHost {
  FaParams p;
  FaTensorMapHost tq, tk, tv, tdo, tdk, tdv;
  float* dq_acc;
  const float* nlse2;
  const float* ndelta;
  int* work_counter;
};

// SMs of the current device (148 on a B200; asked once per device)
int device_sm_count() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  cached[dev].store(n, std::memory_order_relaxed);
  return n;
}

// pairs one item of fa_bwd_tc.cuh may list (fa_btc::MAXPL)
int bwd_tc_max_pairs(int D) { return D == 64 ? 1024 : 2048; }

bool tc_bwd_eligible(const fa_attn_params* p) {
  if (p->flags & FA_FLAG_GENERAL_KERNELS) return false;
  if (p->dtype == FA_F32) return false;
  if (p->D != p->Dv || !(p->D == 64 || p->D == 128)) return false;
  if (p->Sq < 128 || p->Skv < 128) return false;
  // a CTA lists the (query head, q tile) pairs of an item in shared memory: at most 256 q tiles
  // of 128 rows per head, and the pairs of one item must fit the list (a pair is 128 q rows with
  // D = 64, 64 with D = 128)
  const int n_qtiles = (p->Sq + 127) / 128;
  if (n_qtiles > 256) return false;
  if ((long long)n_qtiles * (p->D / 64) * (p->Hq / p->Hkv) > bwd_tc_max_pairs(p->D)) return false;
  const fa_block_tables& t = p->tables;
  if (t.kv_num_blocks) {
    if (!(t.num_q_blocks == 1 || t.q_block_size % 128 == 0)) return false;
    if (!(t.num_kv_blocks == 1 || t.kv_block_size % 128 == 0)) return false;
  }
  return true;
}
size_t delta_bytes(const fa_attn_params* p) { return ((size_t)p->B * p->Hq * p->Sq * sizeof(float) + 255) / 256 * 256; }
size_t rows_pad_bytes(const fa_attn_params* p) {
  const size_t sq_pad = (size_t)((p->Sq + 127) / 128) * 128;
  return ((size_t)p->B * p->Hq * sq_pad * sizeof(float) + 255) / 256 * 256;
}
size_t dq_acc_bytes(const fa_attn_params* p) {
  const size_t sq_pad = (size_t)((p->Sq + 127) / 128) * 128;
  return (size_t)p->B * p->Hq * sq_pad * p->D * sizeof(float);
}

// kv2: two K / V buffers with a three-stage Q / dO ring instead of one with four (head dim 64)
int get_bwd_tc_kernel(fa_module* m, int dtype, int D, int flags, bool kv2, Kernel** k) {
  // must match the shared-memory map of fa_bwd_tc.cuh (fa_btc::SMEM_BYTES)
  const int bq = D == 64 ? 128 : 64, kvbuf = (D == 64 && kv2) ? 2 : 1, nstage = (D == 64 && kvbuf == 1) ? 4 : 3;
  const int kv_bytes = (D / 64) * 16384, q_bytes = 16384, ds_bytes = (bq / 64) * 16384;
  const int smem = 2 * kvbuf * kv_bytes + 2 * nstage * q_bytes + ds_bytes + 128 * 32 * 4 + nstage * 2 * bq * 4 +
                   (2 + 3 * nstage + 15) * 8 + 16 + 16 + 2 * bwd_tc_max_pairs(D) * 4 + 256 + 1024;
  std::string d = defs({{"FA_DTYPE", dtype}, {"FA_D", D}, {"FA_ROUND_SCORES", round_flag(dtype, flags)},
                        {"FA_BWD_KV2", kvbuf == 2 ? 1 : 0}});
  return get_kernel(m, "fa_bwd_tc.cuh", d, "fa_bwd_tc_kernel", smem, k);
}

// With a BlockMask the items are short or uneven and the variant with two K / V buffers wins: under a
// causal mask 97 against 103 us at S=1024 (B16 H8), 150 / 160 at 2048, 197 / 209 at 3072, 263 / 283
// at 4096, 289 / 303 at 6144 (48 q tiles, 24 pairs per item on average).  Without one every item
// has all the q tiles and the four-stage ring wins (S=2048, 16 pairs per item: 206 against 215 us).
bool bwd_tc_kv2(const fa_attn_params* p) {
  if (p->D != 64 || !p->tables.kv_num_blocks) return false;
  return (long long)((p->Sq + 127) / 128) * (p->Hq / p->Hkv) <= 64;
}

int get_mask_bits_kernel(fa_module* m, Kernel** k) {
  return get_kernel(m, "fa_blockmask.cuh", "", "fa_mask_bits_kernel", 0, k);
}

int get_blockmask_kernel(fa_module* m, Kernel** k) {
  return get_kernel(m, "fa_blockmask.cuh", "", "fa_blockmask_classify_kernel", 0, k);
}

}  // namespace

extern "C" {

int fa_module_prepare(fa_module* m, int kind, int dtype, int D, int Dv, int Sq_hint, int Skv_hint) {
  if (!m) return fail(FA_EINVAL, "module is null");
  (void)Skv_hint;
  Kernel* k = nullptr;
  switch (kind) {
    case FA_KIND_FWD: {
      FwdCfg c;
      if (int rc = pick_fwd(dtype, D, Dv, Sq_hint, nullptr, c)) return rc;
      if (dtype != FA_F32 && D == Dv && (D == 64 || D == 128) && Sq_hint >= 128)
        if (int rc = get_fwd_tc_kernel(m, dtype, D, 0, &k)) return rc;
      return get_fwd_kernel(m, dtype, D, Dv, 0, c, &k);
    }
    case FA_KIND_BWD: {
      BwdCfg c;
      if (int rc = pick_bwd(dtype, D, Dv, nullptr, c)) return rc;
      if (dtype != FA_F32 && D == Dv && (D == 64 || D == 128) && Sq_hint >= 128)
        if (int rc = get_bwd_tc_kernel(m, dtype, D, 0, false, &k)) return rc;
        if (D == 64)
          if (int rc = get_bwd_tc_kernel(m, dtype, D, 0, true, &k)) return rc;
      if (int rc = get_bwd_kernel(m, dtype, D, Dv, 0, c, true, &k)) return rc;
      return get_bwd_kernel(m, dtype, D, Dv, 0, c, false, &k);
    }
    case FA_KIND_DECODE: {
      DecCfg c;
      if (int rc = pick_decode(dtype, D, Dv, Sq_hint, nullptr, c)) return rc;
      if (dtype != FA_F32 && D == 64 && Dv == 64 && Sq_hint >= 2)
        if (int rc = get_fwd_tc_kernel(m, dtype, D, 0, &k, true)) return rc;
      return get_decode_kernel(m, dtype, D, Dv, 0, c, false, &k);
    }
    case FA_KIND_BLOCKMASK:
      if (int rc = get_mask_bits_kernel(m, &k)) return rc;
      return get_blockmask_kernel(m, &k);
    default:
      return fail(FA_EUNSUPPORTED, "fa_module_prepare: unknown kind");
  }
}

int fa_fwd(fa_module* m, const fa_attn_params* p, void* stream) {
  if (int rc = check_common(m, p)) return rc;
  prof_reset();
  FaParams kp;
  fill_params(p, kp);
  if (tc_fwd_eligible(p)) return launch_fwd_tc(m, p, kp, stream);
  FwdCfg c;
  if (int rc = pick_fwd(p->dtype, p->D, p->Dv, p->Sq, &kp.t, c)) return rc;
  Kernel* k = nullptr;
  if (int rc = get_fwd_kernel(m, p->dtype, p->D, p->Dv, p->flags, c, &k)) return rc;
  kp.n_q_tiles = (p->Sq + c.BM - 1) / c.BM;
  return launch(k, dim3(kp.n_q_tiles, p->Hq, p->B), dim3(c.warps * 32), &kp, stream);
}

size_t fa_bwd_workspace_bytes(const fa_attn_params* p) {
  if (!p || p->B <= 0 || p->Hq <= 0 || p->Sq <= 0) return 0;
  if (p->Hkv > 0 && p->Hq % p->Hkv == 0 && tc_bwd_eligible(p)) return 2 * rows_pad_bytes(p) + dq_acc_bytes(p) + 256;
  return delta_bytes(p);
}

int fa_bwd(fa_module* m, const fa_attn_params* p, const fa_tensor* dout, const fa_tensor* dq, const fa_tensor* dk,
           const fa_tensor* dv, void* workspace, size_t workspace_bytes, void* stream) {
  if (int rc = check_common(m, p)) return rc;
  if (!dout || !dq || !dk || !dv) return fail(FA_EINVAL, "dout, dq, dk and dv descriptors are required");
  const int es = esize(p->dtype);
  if (int rc = check_tensor(*dout, "dout", es)) return rc;
  if (int rc = check_tensor(*dq, "dq", es)) return rc;
  if (int rc = check_tensor(*dk, "dk", es)) return rc;
  if (int rc = check_tensor(*dv, "dv", es)) return rc;
  if (!p->lse) return fail(FA_EINVAL, "lse (forward logsumexp) is required for the backward pass");
  if (p->tables.kv_num_blocks && !p->tables.q_num_blocks)
    return fail(FA_EINVAL, "the backward pass needs the q tables of the BlockMask");
  if (p->tables.kv_num_blocks && ((p->tables.full_q_num_blocks == nullptr) != (p->tables.full_kv_num_blocks == nullptr)))
    return fail(FA_EINVAL, "full q tables and full kv tables must be given together");
  const size_t need = fa_bwd_workspace_bytes(p);
  if (!workspace || workspace_bytes < need) return fail(FA_EWORKSPACE, "backward workspace too small");
  prof_reset();
  FaParams kp;
  fill_params(p, kp);
  kp.dout = cvt(*dout); kp.dq = cvt(*dq); kp.dk = cvt(*dk); kp.dv = cvt(*dv);
  kp.delta = (float*)workspace;
  const bool use_tc = tc_bwd_eligible(p);
  BwdCfg c{};
  Kernel *kdq = nullptr, *kdkdv = nullptr, *ktc = nullptr;
  if (use_tc) {
    if (int rc = get_bwd_tc_kernel(m, p->dtype, p->D, p->flags, bwd_tc_kv2(p), &ktc)) return rc;
  } else {
    if (int rc = pick_bwd(p->dtype, p->D, p->Dv, &kp.t, c)) return rc;
    if (int rc = get_bwd_kernel(m, p->dtype, p->D, p->Dv, p->flags, c, true, &kdq)) return rc;
    if (int rc = get_bwd_kernel(m, p->dtype, p->D, p->Dv, p->flags, c, false, &kdkdv)) return rc;
  }
  if (use_tc) {
    // workspace: nlse2 | ndelta (padded rows) | dq accumulator
    cudaStream_t st = (cudaStream_t)stream;
    float* nlse2 = (float*)workspace;
    float* ndelta = (float*)((char*)workspace + rows_pad_bytes(p));
    float* dq_acc = (float*)((char*)workspace + 2 * rows_pad_bytes(p));
    int* work_counter = (int*)((char*)workspace + 2 * rows_pad_bytes(p) + dq_acc_bytes(p));  // zeroed by the prep kernel
    const int sq_pad = (p->Sq + 127) / 128 * 128;
    const int n_bh = p->B * p->Hq;
    const int gy = n_bh < 32768 ? n_bh : 32768;
    {
      // row scalars; the same pass clears the dQ accumulator
      // 8 lanes per row, 4 rows per thread: 128 rows per block (sq_pad is a multiple of 128)
      const dim3 grid((unsigned)(sq_pad / 128), (unsigned)gy, (unsigned)((n_bh + gy - 1) / gy));
      ProfScope prof("fa_bwd_prep_kernel", stream);
      if (p->dtype == FA_F16)
        fa_bwd_prep_kernel<FA_F16, 8><<<grid, 256, 0, st>>>(kp.o, kp.dout, p->lse, nlse2, ndelta, dq_acc, work_counter, p->Hq, p->Sq, sq_pad, p->Dv, p->D, n_bh);
      else
        fa_bwd_prep_kernel<FA_BF16, 8><<<grid, 256, 0, st>>>(kp.o, kp.dout, p->lse, nlse2, ndelta, dq_acc, work_counter, p->Hq, p->Sq, sq_pad, p->Dv, p->D, n_bh);
      FA_CUDA_CHECK(cudaGetLastError());
    }
    FaBwdTcParamsHost tp;
    tp.p = kp;
    tp.dq_acc = dq_acc;
    tp.nlse2 = nlse2;
    tp.ndelta = ndelta;
    tp.work_counter = work_counter;
    const int bq = p->D == 64 ? 128 : 64;  // q rows of a (kv tile, q tile) pair of the kernel
    if (int rc = make_map(&tp.tq, p->dtype, p->q, p->D, p->Sq, p->Hq, p->B, bq)) return rc;
    if (int rc = make_map(&tp.tk, p->dtype, p->k, p->D, p->Skv, p->Hkv, p->B)) return rc;
    if (int rc = make_map(&tp.tv, p->dtype, p->v, p->Dv, p->Skv, p->Hkv, p->B)) return rc;
    if (int rc = make_map(&tp.tdo, p->dtype, *dout, p->Dv, p->Sq, p->Hq, p->B, bq)) return rc;
    if (int rc = make_map(&tp.tdk, p->dtype, *dk, p->D, p->Skv, p->Hkv, p->B)) return rc;
    if (int rc = make_map(&tp.tdv, p->dtype, *dv, p->Dv, p->Skv, p->Hkv, p->B)) return rc;
    // persistent: one CTA per SM (fewer when there are fewer items), items handed out through the counter
    const long long n_items = (long long)p->Hkv * p->B * ((p->Skv + 127) / 128);
    if (int rc = launch(ktc, dim3((unsigned)std::min<long long>(n_items, device_sm_count())), dim3(512), &tp, stream)) return rc;
    {
      // one 16-byte output chunk per thread: D / 8 chunks per row
      const dim3 grid((unsigned)(((long long)sq_pad * (p->D / 8) + 255) / 256), (unsigned)gy, (unsigned)((n_bh + gy - 1) / gy));
      ProfScope prof("fa_dq_convert_kernel", stream);
      if (p->D == 64) {
        if (p->dtype == FA_F16)
          fa_dq_convert_kernel<FA_F16><<<grid, 256, 0, st>>>(dq_acc, kp.dq, p->Hq, p->Sq, sq_pad, p->scale, n_bh);
        else
          fa_dq_convert_kernel<FA_BF16><<<grid, 256, 0, st>>>(dq_acc, kp.dq, p->Hq, p->Sq, sq_pad, p->scale, n_bh);
      } else {
        if (p->dtype == FA_F16)
          fa_dq_convert_t_kernel<FA_F16><<<grid, 256, 0, st>>>(dq_acc, kp.dq, p->Hq, p->Sq, sq_pad, p->scale, n_bh);
        else
          fa_dq_convert_t_kernel<FA_BF16><<<grid, 256, 0, st>>>(dq_acc, kp.dq, p->Hq, p->Sq, sq_pad, p->scale, n_bh);
      }
      FA_CUDA_CHECK(cudaGetLastError());
    }
    return FA_OK;
  }
  {
    cudaStream_t st = (cudaStream_t)stream;
    const long long n_rows = (long long)p->B * p->Hq * p->Sq;
    const int chunks = p->Dv * es / 16;
    const int lpr = chunks >= 8 ? 8 : (chunks >= 4 ? 4 : (chunks >= 2 ? 2 : 1));
    const long long threads = n_rows * lpr;
    const unsigned blocks = (unsigned)((threads + 255) / 256);
    ProfScope prof("fa_delta_kernel", stream);
#define FA_DELTA(DT, L) fa_delta_kernel<DT, L><<<blocks, 256, 0, st>>>(kp.o, kp.dout, kp.delta, p->Hq, p->Sq, p->Dv, n_rows)
#define FA_DELTA_DT(L)                                      \
  do {                                                      \
    if (p->dtype == FA_F16) FA_DELTA(FA_F16, L);            \
    else if (p->dtype == FA_BF16) FA_DELTA(FA_BF16, L);     \
    else FA_DELTA(FA_F32, L);                               \
  } while (0)
    if (lpr == 8) FA_DELTA_DT(8);
    else if (lpr == 4) FA_DELTA_DT(4);
    else if (lpr == 2) FA_DELTA_DT(2);
    else FA_DELTA_DT(1);
#undef FA_DELTA_DT
#undef FA_DELTA
    FA_CUDA_CHECK(cudaGetLastError());
  }
  if (int rc = launch(kdkdv, dim3((p->Skv + c.tile - 1) / c.tile, p->Hkv, p->B), dim3(c.warps * 32), &kp, stream))
    return rc;
  return launch(kdq, dim3((p->Sq + c.tile - 1) / c.tile, p->Hq, p->B), dim3(c.warps * 32), &kp, stream);
}

// Smallest number of CTAs per (batch, head), up to cmax, whose grid fills its last wave of `slots`
// concurrent CTAs to 95 %; the best found if none does.
static int fill_waves(long long bh, int cmax, int slots) {
  int best = 1;
  double best_eff = 0.0;
  for (int c = 1; c <= cmax; ++c) {
    const double waves = (double)(bh * c) / slots;
    const double eff = waves / (double)(long long)(waves + 0.999999);
    if (eff >= 0.95) return c;
    if (eff > best_eff + 1e-9) {
      best_eff = eff;
      best = c;
    }
  }
  return best;
}

int fa_decode_packs_heads(const fa_attn_params* p) { return (p && decode_packs_heads(p)) ? 1 : 0; }

int fa_decode_num_splits(const fa_attn_params* p, int sm_count) {
  if (!p || p->B <= 0 || p->Hq <= 0 || p->Skv <= 0) return 1;
  if (sm_count <= 0) sm_count = 148;
  const bool pack = decode_packs_heads(p);
  const long long bh = (long long)p->B * (pack ? p->Hkv : p->Hq);
  const int tiles = (p->Skv + 127) / 128;
  if (!pack && tc_decode_eligible(p)) {
    // tcgen05 kernel: one CTA per SM and split, at least eight kv tiles per CTA; its partial results
    // always go through the combine kernel, so there are at least two splits
    const int cmax = tiles / 8 > 1 ? (tiles / 8 < 64 ? tiles / 8 : 64) : 1;
    const int c = fill_waves(bh, cmax, sm_count);
    return c < 2 ? 2 : c;
  }
  // general kernel: as many CTAs per SM as its shared memory allows (at most four by registers),
  // at least four kv tiles per CTA.  A grid that ends in a part-filled wave costs more than a few
  // extra partial results.
  int per_sm = 2;
  DecCfg c;
  if (pick_decode(p->dtype, p->D, p->Dv, pack ? p->Sq * (p->Hq / p->Hkv) : p->Sq, nullptr, c) == FA_OK) {
    per_sm = (228 * 1024) / (c.smem + 1024);
    per_sm = per_sm < 1 ? 1 : (per_sm > 4 ? 4 : per_sm);
  }
  const int cmax = tiles / 4 > 1 ? (tiles / 4 < 64 ? tiles / 4 : 64) : 1;
  return fill_waves(bh, cmax, per_sm * sm_count);
}

size_t fa_decode_workspace_bytes(const fa_attn_params* p, int num_splits) {
  if (!p || num_splits <= 1) return 0;
  const size_t rows = (size_t)p->B * p->Hq * num_splits * p->Sq;
  return (rows * p->Dv * sizeof(float) + 255) / 256 * 256 + (rows * 2 * sizeof(float) + 255) / 256 * 256;
}

int fa_decode(fa_module* m, const fa_attn_params* p, int num_splits, void* workspace, size_t workspace_bytes,
              void* stream) {
  if (int rc = check_common(m, p)) return rc;
  if (num_splits <= 0) num_splits = fa_decode_num_splits(p, 0);
  if (num_splits > 65535) return fail(FA_EINVAL, "too many splits");
  prof_reset();
  FaParams kp;
  fill_params(p, kp);
  const bool pack = decode_packs_heads(p);
  const bool tc = !pack && tc_decode_eligible(p) && num_splits >= 2;
  DecCfg c;
  if (!tc)
    if (int rc = pick_decode(p->dtype, p->D, p->Dv, pack ? p->Sq * (p->Hq / p->Hkv) : p->Sq, &kp.t, c)) return rc;
  const size_t need = fa_decode_workspace_bytes(p, num_splits);
  if (need && (!workspace || workspace_bytes < need)) return fail(FA_EWORKSPACE, "decode workspace too small");
  if (need && ((uintptr_t)workspace & 15)) return fail(FA_EINVAL, "workspace must be 16-byte aligned");
  kp.num_splits = num_splits;
  if (need) {
    const size_t rows = (size_t)p->B * p->Hq * num_splits * p->Sq;
    kp.part_o = (float*)workspace;
    kp.part_ml = (float*)((char*)workspace + (rows * p->Dv * sizeof(float) + 255) / 256 * 256);
  }
  if (tc) {
    // tcgen05 kernel: num_splits CTAs per (batch, head), each writing one partial result per row
    if (int rc = launch_decode_tc(m, p, kp, num_splits, stream)) return rc;
  } else {
    Kernel* k = nullptr;
    if (int rc = get_decode_kernel(m, p->dtype, p->D, p->Dv, p->flags, c, pack, &k)) return rc;
    if (int rc = launch(k, dim3(num_splits, pack ? p->Hkv : p->Hq, p->B), dim3(128), &kp, stream)) return rc;
  }
  if (num_splits > 1) {
    const long long n_rows = (long long)p->B * p->Hq * p->Sq;
    const unsigned blocks = (unsigned)((n_rows + 3) / 4);
    cudaStream_t st = (cudaStream_t)stream;
    ProfScope prof("fa_decode_combine_kernel", stream);
    if (p->dtype == FA_F16)
      fa_decode_combine_kernel<FA_F16><<<blocks, 128, 0, st>>>(kp.part_o, kp.part_ml, kp.o, kp.lse, p->Hq, p->Sq, p->Dv, num_splits, n_rows);
    else
      fa_decode_combine_kernel<FA_BF16><<<blocks, 128, 0, st>>>(kp.part_o, kp.part_ml, kp.o, kp.lse, p->Hq, p->Sq, p->Dv, num_splits, n_rows);
    FA_CUDA_CHECK(cudaGetLastError());
  }
  return FA_OK;
}

size_t fa_block_mask_workspace_bytes(int B, int H, int Q_LEN, int KV_LEN, int q_block, int kv_block) {
  if (B <= 0 || H <= 0 || Q_LEN <= 0 || KV_LEN <= 0 || q_block <= 0 || kv_block <= 0) return 0;
  const long long nQ = (Q_LEN + q_block - 1) / q_block, nKV = (KV_LEN + kv_block - 1) / kv_block;
  return (size_t)((long long)B * H * nQ * nKV);
}

int64_t fa_mask_bits_row_words(int KV_LEN) { return KV_LEN <= 0 ? 0 : (int64_t)((KV_LEN + 127) / 128) * 4; }

int fa_mask_bits(fa_module* m, int B, int H, int Q_LEN, int KV_LEN, int b_offset, int h_offset, uint32_t* bits,
                 void* stream) {
  if (!m) return fail(FA_EINVAL, "module is null");
  if (B <= 0 || H <= 0 || Q_LEN <= 0 || KV_LEN <= 0) return fail(FA_EINVAL, "B, H, Q_LEN and KV_LEN must be positive");
  if (!bits || ((uintptr_t)bits & 15)) return fail(FA_EINVAL, "bits must be a 16-byte aligned device pointer");
  if ((long long)B * H > 65535 || Q_LEN > 65535) return fail(FA_EUNSUPPORTED, "B*H and Q_LEN must not exceed 65535");
  Kernel* k = nullptr;
  if (int rc = get_mask_bits_kernel(m, &k)) return rc;
  FaMaskBitsParams mp;
  mp.bits = bits;
  mp.stride = fa_mask_bits_row_words(KV_LEN);
  mp.B = B; mp.H = H; mp.Q_LEN = Q_LEN; mp.KV_LEN = KV_LEN;
  mp.b_off = b_offset; mp.h_off = h_offset;
  return launch(k, dim3((unsigned)((mp.stride + 255) / 256), (unsigned)Q_LEN, (unsigned)(B * H)), dim3(256), &mp, stream);
}

int fa_block_mask(fa_module* m, int B, int H, int Q_LEN, int KV_LEN, int q_block, int kv_block, int b_offset,
                  int h_offset, int32_t* kv_num_blocks, int32_t* kv_indices, int32_t* full_kv_num_blocks,
                  int32_t* full_kv_indices, int32_t* q_num_blocks, int32_t* q_indices, int32_t* full_q_num_blocks,
                  int32_t* full_q_indices, void* workspace, size_t workspace_bytes, void* stream) {
  if (!m) return fail(FA_EINVAL, "module is null");
  const size_t need = fa_block_mask_workspace_bytes(B, H, Q_LEN, KV_LEN, q_block, kv_block);
  if (need == 0) return fail(FA_EINVAL, "B, H, Q_LEN, KV_LEN and block sizes must be positive");
  if (!kv_num_blocks || !kv_indices) return fail(FA_EINVAL, "kv_num_blocks / kv_indices are null");
  if ((full_kv_num_blocks == nullptr) != (full_kv_indices == nullptr))
    return fail(FA_EINVAL, "full_kv_num_blocks and full_kv_indices must be both given or both null");
  if ((q_num_blocks == nullptr) != (q_indices == nullptr) || (full_q_num_blocks == nullptr) != (full_q_indices == nullptr))
    return fail(FA_EINVAL, "q tables must be given as (num, indices) pairs");
  if (full_q_num_blocks && !full_kv_num_blocks) return fail(FA_EINVAL, "full q tables need full kv tables");
  if (!workspace || workspace_bytes < need) return fail(FA_EWORKSPACE, "block-mask workspace too small");
  const int nQ = (Q_LEN + q_block - 1) / q_block, nKV = (KV_LEN + kv_block - 1) / kv_block;
  if ((long long)B * H > 65535 || nQ > 65535) return fail(FA_EUNSUPPORTED, "B*H and the q-block count must not exceed 65535");
  Kernel* k = nullptr;
  if (int rc = get_blockmask_kernel(m, &k)) return rc;
  FaMaskParams mp;
  mp.cls = (signed char*)workspace;
  mp.B = B; mp.H = H; mp.nQ = nQ; mp.nKV = nKV; mp.QB = q_block; mp.KVB = kv_block;
  mp.b_off = b_offset; mp.h_off = h_offset;
  if (int rc = launch(k, dim3(nKV, nQ, B * H), dim3(256), &mp, stream)) return rc;

  cudaStream_t st = (cudaStream_t)stream;
  const int wpb = 4;
  auto run = [&](int want, bool transposed, int32_t* num, int32_t* idx) -> int {
    if (!num) return FA_OK;
    const int rows = transposed ? nKV : nQ, cols = transposed ? nQ : nKV;
    const long long n_rows = (long long)B * H * rows;
    const unsigned blocks = (unsigned)((n_rows + wpb - 1) / wpb);
    fa_tables_kernel<<<blocks, wpb * 32, 0, st>>>(mp.cls, rows, cols, want, transposed, nQ, nKV, n_rows, num, idx);
    FA_CUDA_CHECK(cudaGetLastError());
    return FA_OK;
  };
  // Without separate full tables every non-empty block is listed as partial.
  if (!full_kv_num_blocks) return fail(FA_EUNSUPPORTED, "tables without separate full blocks are not implemented");
  if (int rc = run(1, false, kv_num_blocks, kv_indices)) return rc;
  if (int rc = run(2, false, full_kv_num_blocks, full_kv_indices)) return rc;
  if (int rc = run(1, true, q_num_blocks, q_indices)) return rc;
  if (int rc = run(2, true, full_q_num_blocks, full_q_indices)) return rc;
  return FA_OK;
}

}  // extern "C"

// ======================================================================================
// Decode without any allocation by the caller or the library
// ======================================================================================
namespace {

// Scratch for the split-KV partial results of fa_decode_static.  It is part of the loaded
// library image: every GPU that loads the library holds these bytes until the process exits.
constexpr size_t kStaticScratchBytes = (size_t)FA_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_static_mu;
void* g_static_ptr[64] = {nullptr};

// In host code `g_static_scratch` is only a handle for the symbol, not a device address; the
// address a kernel can use has to be asked for, once per device, with that device current.
int static_scratch(void** out, void* stream) {
  int dev = 0;
  FA_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(FA_EUNSUPPORTED, "device ordinal above 63");
  // the scratch address is the current device's: a stream of another device would run the kernels there
  if (stream != nullptr && stream != (void*)cudaStreamLegacy && stream != (void*)cudaStreamPerThread) {
    int sdev = dev;
    if (cudaStreamGetDevice((cudaStream_t)stream, &sdev) == cudaSuccess && sdev != dev)
      return fail(FA_EINVAL, "fa_decode_static: the stream belongs to device " + std::to_string(sdev) +
                                 ", the current device is " + std::to_string(dev));
    cudaGetLastError();
  }
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    FA_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_static_scratch));
    if (ptr == nullptr) return fail(FA_ECUDA, "cudaGetSymbolAddress returned a null address");
    g_static_ptr[dev] = ptr;
  }
  *out = g_static_ptr[dev];
  return FA_OK;
}

}  // namespace

extern "C" {

size_t fa_decode_static_capacity(void) { return kStaticScratchBytes; }

int fa_decode_static(fa_module* m, const fa_attn_params* p, int num_splits, void* stream) {
  // arguments first: the sizes below are products of fields that have to be positive
  if (int rc = check_common(m, p)) return rc;
  if (p->dtype == FA_F32) return fail(FA_EUNSUPPORTED, "the decode kernel takes fp16 / bf16 inputs");
  if (p->Sq > 64) return fail(FA_EUNSUPPORTED, "the decode kernel handles at most 64 query rows");
  if (num_splits <= 0) num_splits = fa_decode_num_splits(p, 0);
  const size_t need = fa_decode_workspace_bytes(p, num_splits);
  if (need == 0) return fa_decode(m, p, num_splits, nullptr, 0, stream);  // a single split needs no scratch
  if (need > kStaticScratchBytes)
    return fail(FA_EWORKSPACE, "fa_decode_static: this problem needs " + std::to_string(need) +
                                   " bytes of split-KV scratch, the built-in scratch holds " +
                                   std::to_string(kStaticScratchBytes) + "; use fewer splits or fa_decode");
  void* ws = nullptr;
  if (int rc = static_scratch(&ws, stream)) return rc;
  return fa_decode(m, p, num_splits, ws, kStaticScratchBytes, stream);
}

}  // extern "C"
