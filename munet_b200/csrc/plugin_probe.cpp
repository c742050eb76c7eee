// libmunet_backend_b200.so — the probe MuNet's plugin loader looks for before it
// enables its CUDA device slot (src/backend/plugin_loader.cpp:101-176, ABI
// constant src/backend/plugin_loader.hpp:9; shipped example
// src/backend/plugins/plugin_cu12.cpp:1-9). The loader dlopens every
// `libmunet_backend_*.so` it finds, calls these five symbols and dlcloses it
// again: the plugin is a gate, not a code path. Strings have static storage.
//
// The probe succeeds when the NVIDIA driver library and the kernel library that
// sits next to this file can be loaded and the kernel library reports the ABI
// this probe was built for.
#include <cstdint>
#include <cstdio>
#include <dlfcn.h>
#include <string>

namespace {
char g_error[512];

std::string own_directory() {
  Dl_info info;
  if (dladdr(reinterpret_cast<const void *>(&own_directory), &info) && info.dli_fname) {
    std::string p(info.dli_fname);
    const size_t slash = p.find_last_of('/');
    return slash == std::string::npos ? std::string(".") : p.substr(0, slash);
  }
  return ".";
}
} // namespace

extern "C" {

uint32_t munet_backend_plugin_abi_version(void) { return 1u; }
const char *munet_backend_plugin_name(void) { return "b200"; }
const char *munet_backend_plugin_device_type(void) { return "cuda"; }
// same six capability bits the reference's CUDA plugins advertise (0x3F)
uint64_t munet_backend_plugin_capability_flags(void) { return 0x3Fu; }

const char *munet_backend_plugin_probe(void) {
  void *drv = dlopen("libcuda.so.1", RTLD_LAZY | RTLD_LOCAL);
  if (!drv) {
    snprintf(g_error, sizeof(g_error), "Missing runtime dependency: libcuda.so.1");
    return g_error;
  }
  dlclose(drv);
  const std::string lib = own_directory() + "/libmunet_b200.so";
  void *h = dlopen(lib.c_str(), RTLD_LAZY | RTLD_LOCAL);
  if (!h) {
    const char *why = dlerror();
    snprintf(g_error, sizeof(g_error), "Missing runtime dependency: %s (%s)", lib.c_str(),
             why ? why : "dlopen failed");
    return g_error;
  }
  using VersionFn = int (*)();
  VersionFn version = reinterpret_cast<VersionFn>(dlsym(h, "mu_abi_version"));
  const int v = version ? version() : -1;
  dlclose(h);
  if (v != 1) {
    snprintf(g_error, sizeof(g_error), "libmunet_b200.so reports ABI %d, this probe needs 1", v);
    return g_error;
  }
  return nullptr;
}

} // extern "C"
