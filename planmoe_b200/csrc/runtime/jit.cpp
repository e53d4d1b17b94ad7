#include "runtime/jit.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nvrtc.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <pybind11/stl.h>

#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

namespace py = pybind11;

namespace {

struct Nvrtc {
  decltype(&nvrtcCreateProgram) create = nullptr;
  decltype(&nvrtcCompileProgram) compile = nullptr;
  decltype(&nvrtcGetCUBINSize) cubin_size = nullptr;
  decltype(&nvrtcGetCUBIN) cubin = nullptr;
  decltype(&nvrtcGetProgramLogSize) log_size = nullptr;
  decltype(&nvrtcGetProgramLog) log = nullptr;
  decltype(&nvrtcDestroyProgram) destroy = nullptr;
  decltype(&nvrtcGetErrorString) err = nullptr;
};

Nvrtc& nvrtc() {
  static Nvrtc n;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so.12", "libnvrtc.so",
                           "/usr/local/cuda/lib64/libnvrtc.so"};
    void* h = nullptr;
    for (const char* nm : names) {
      h = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
      if (h != nullptr) break;
    }
    if (h == nullptr) throw std::runtime_error("planmoe jit: libnvrtc not found");
#define LOAD(field, sym) n.field = reinterpret_cast<decltype(n.field)>(dlsym(h, sym))
    LOAD(create, "nvrtcCreateProgram");
    LOAD(compile, "nvrtcCompileProgram");
    LOAD(cubin_size, "nvrtcGetCUBINSize");
    LOAD(cubin, "nvrtcGetCUBIN");
    LOAD(log_size, "nvrtcGetProgramLogSize");
    LOAD(log, "nvrtcGetProgramLog");
    LOAD(destroy, "nvrtcDestroyProgram");
    LOAD(err, "nvrtcGetErrorString");
#undef LOAD
  });
  return n;
}

template <class F>
F driver_fn(const char* name) {
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &sym, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    throw std::runtime_error(std::string("planmoe jit: driver entry point not available: ") + name);
  return reinterpret_cast<F>(sym);
}

struct Kernel {
  std::string source, name, cubin;
  std::map<int, CUfunction> per_device;
};

std::vector<Kernel>& kernels() {
  static std::vector<Kernel> k;
  return k;
}

std::string g_sdk_home = "/usr/local/cuda";

// nvcc route: write the source to a temporary file and run `<sdk>/bin/nvcc --cubin` as a child process
// (the reference's default route, PlanMoE/custom/jit.h:87-118, with its -gencode derived from the live
// device; here the target is always sm_100a).  Used when USE_NVRTC=0 or libnvrtc cannot be loaded.
std::string compile_cubin_nvcc(const std::string& source, const std::string& name) {
  char src_path[] = "/tmp/planmoe_jit_XXXXXX.cu";
  const int fd = mkstemps(src_path, 3);
  if (fd < 0) throw std::runtime_error("planmoe jit: cannot create a temporary source file");
  const std::string cubin_path = std::string(src_path) + ".cubin";
  const std::string log_path = std::string(src_path) + ".log";
  {
    FILE* f = fdopen(fd, "w");
    if (f == nullptr) { close(fd); throw std::runtime_error("planmoe jit: cannot open the temporary source file"); }
    fwrite(source.data(), 1, source.size(), f);
    fclose(f);
  }
  const std::string cmd = "'" + g_sdk_home + "/bin/nvcc' --cubin -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 "
                          "--use_fast_math -o '" + cubin_path + "' '" + src_path + "' > '" + log_path + "' 2>&1";
  const int rc = std::system(cmd.c_str());
  auto slurp = [](const std::string& path) {
    std::string out;
    if (FILE* f = fopen(path.c_str(), "rb")) {
      char buf[4096];
      size_t got;
      while ((got = fread(buf, 1, sizeof(buf), f)) > 0) out.append(buf, got);
      fclose(f);
    }
    return out;
  };
  std::string cubin = rc == 0 ? slurp(cubin_path) : std::string();
  const std::string log = slurp(log_path);
  unlink(src_path); unlink(cubin_path.c_str()); unlink(log_path.c_str());
  if (rc != 0 || cubin.empty())
    throw std::runtime_error("planmoe jit: nvcc failed for kernel `" + name + "`:\n" + log);
  return cubin;
}

bool want_nvrtc() {
  const char* e = getenv("USE_NVRTC");
  return !(e != nullptr && e[0] == '0');
}

std::string compile_cubin(const std::string& source, const std::string& name) {
  if (!want_nvrtc()) return compile_cubin_nvcc(source, name);
  Nvrtc* np = nullptr;
  try {
    np = &nvrtc();
  } catch (const std::exception&) {
    return compile_cubin_nvcc(source, name);       // no libnvrtc on this machine: fall back to nvcc
  }
  Nvrtc& n = *np;
  nvrtcProgram prog;
  if (n.create(&prog, source.c_str(), (name + ".cu").c_str(), 0, nullptr, nullptr) != NVRTC_SUCCESS)
    throw std::runtime_error("nvrtcCreateProgram failed");
  const std::string inc = "-I" + g_sdk_home + "/include";
  const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "--use_fast_math", inc.c_str()};
  nvrtcResult r = n.compile(prog, 4, opts);
  if (r != NVRTC_SUCCESS) {
    size_t ls = 0;
    n.log_size(prog, &ls);
    std::string log(ls, '\0');
    if (ls > 0) n.log(prog, &log[0]);
    n.destroy(&prog);
    throw std::runtime_error("planmoe jit: compilation failed:\n" + log);
  }
  size_t sz = 0;
  n.cubin_size(prog, &sz);
  std::string cubin(sz, '\0');
  n.cubin(prog, &cubin[0]);
  n.destroy(&prog);
  return cubin;
}

void update_sdk_home(const std::string& home) { g_sdk_home = home; }

// Registers a kernel; compilation happens at the first invoke (needs only NVRTC, no GPU).
int inject_source(const std::string& source, const std::string& name) {
  Kernel k;
  k.source = "extern \"C\" " + source;
  // keep user-provided extern "C" declarations intact
  if (source.find("extern \"C\"") != std::string::npos) k.source = source;
  k.name = name;
  kernels().push_back(std::move(k));
  return (int)kernels().size() - 1;
}

std::string compile_only(int fd) {
  Kernel& k = kernels().at(fd);
  if (k.cubin.empty()) k.cubin = compile_cubin(k.source, k.name);
  return std::to_string(k.cubin.size());
}

void invoke(int fd, const std::vector<unsigned long long>& pointers, const std::vector<long long>& scalars,
            const std::vector<int>& grid, const std::vector<int>& block, unsigned long long stream) {
  Kernel& k = kernels().at(fd);
  if (k.cubin.empty()) k.cubin = compile_cubin(k.source, k.name);
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) throw std::runtime_error("planmoe jit: no CUDA device");
  cudaFree(nullptr);   // make sure the primary context is current
  auto it = k.per_device.find(dev);
  if (it == k.per_device.end()) {
    static auto load = driver_fn<CUresult (*)(CUmodule*, const void*)>("cuModuleLoadData");
    static auto getfn = driver_fn<CUresult (*)(CUfunction*, CUmodule, const char*)>("cuModuleGetFunction");
    CUmodule mod;
    if (load(&mod, k.cubin.data()) != CUDA_SUCCESS) throw std::runtime_error("planmoe jit: cuModuleLoadData failed");
    CUfunction fn;
    if (getfn(&fn, mod, k.name.c_str()) != CUDA_SUCCESS)
      throw std::runtime_error("planmoe jit: kernel `" + k.name + "` not found in module");
    it = k.per_device.emplace(dev, fn).first;
  }
  static auto launch = driver_fn<CUresult (*)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                                              unsigned, CUstream, void**, void**)>("cuLaunchKernel");
  std::vector<unsigned long long> ptrs = pointers;
  std::vector<int> ints(scalars.begin(), scalars.end());
  std::vector<void*> args;
  for (auto& p : ptrs) args.push_back(&p);
  for (auto& s : ints) args.push_back(&s);
  auto dim = [](const std::vector<int>& v, size_t i) { return (unsigned)(i < v.size() && v[i] > 0 ? v[i] : 1); };
  CUresult r = launch(it->second, dim(grid, 0), dim(grid, 1), dim(grid, 2), dim(block, 0), dim(block, 1), dim(block, 2),
                      0, reinterpret_cast<CUstream>(stream), args.data(), nullptr);
  if (r != CUDA_SUCCESS) throw std::runtime_error("planmoe jit: cuLaunchKernel failed with code " + std::to_string((int)r));
}

}  // namespace

void bind_jit(py::module_& m) {
  m.def("update_sdk_home", &update_sdk_home);
  m.def("jit_inject_source_raw", &inject_source);
  m.def("jit_compile", &compile_only);
  m.def("jit_invoke_raw", &invoke);
}
