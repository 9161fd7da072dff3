// Locked PID file and NVML topology enumeration (see bus.h for the declarations).
//
// Pidfile: open(O_CREAT) + flock(LOCK_EX | LOCK_NB); a second process gets "AlreadyRunning:<pid>"
// (the reference binds libbsd's pidfile through Rust: rust/exo_rs/src/pidfile.rs:58-124).
// NVML: the library is loaded with dlopen at run time, so the module imports on machines without
// a driver; this replaces the reference's Thunderbolt / RDMA probing
// (src/exo/utils/info_gatherer/info_gatherer.py) as the source of link topology.
#include <dlfcn.h>
#include <errno.h>
#include <fcntl.h>
#include <string.h>
#include <sys/file.h>
#include <unistd.h>

#include <stdexcept>

#include "bus.h"

namespace exo {

Pidfile::Pidfile(const std::string& path) : path_(path) {
  fd_ = ::open(path.c_str(), O_RDWR | O_CREAT | O_CLOEXEC, 0644);
  if (fd_ < 0) throw std::runtime_error(std::string("cannot open pidfile: ") + strerror(errno));
  if (::flock(fd_, LOCK_EX | LOCK_NB) != 0) {
    char buf[32] = {0};
    ssize_t n = ::pread(fd_, buf, sizeof buf - 1, 0);
    ::close(fd_);
    fd_ = -1;
    long pid = n > 0 ? strtol(buf, nullptr, 10) : 0;
    throw std::runtime_error("AlreadyRunning:" + std::to_string(pid));
  }
  if (::ftruncate(fd_, 0) != 0) { /* keep going: write() rewrites from offset 0 */ }
}

void Pidfile::write() {
  if (fd_ < 0) throw std::runtime_error("pidfile is closed");
  std::string s = std::to_string((long)getpid()) + "\n";
  if (::ftruncate(fd_, 0) != 0 || ::pwrite(fd_, s.data(), s.size(), 0) != (ssize_t)s.size())
    throw std::runtime_error(std::string("cannot write pidfile: ") + strerror(errno));
  ::fsync(fd_);
}

void Pidfile::close() {
  if (fd_ < 0) return;
  ::unlink(path_.c_str());
  ::flock(fd_, LOCK_UN);
  ::close(fd_);
  fd_ = -1;
}

Pidfile::~Pidfile() { close(); }

// ---- NVML (minimal prototypes; types kept opaque) ----------------------------------------------
namespace {
typedef void* nvmlDevice_t;
struct nvmlMemory_t { unsigned long long total, free, used; };
struct nvmlUtilization_t { unsigned gpu, memory; };
struct nvmlPciInfo_t { char busIdLegacy[16]; unsigned domain, bus, device, pciDeviceId, pciSubSystemId; char busId[32]; };
constexpr int NVML_LINKS = 18;

template <typename F> F sym(void* h, const char* n) { return reinterpret_cast<F>(dlsym(h, n)); }
}  // namespace

std::vector<GpuInfo> nvml_enumerate(std::string* error) {
  std::vector<GpuInfo> out;
  void* h = dlopen("libnvidia-ml.so.1", RTLD_NOW | RTLD_LOCAL);
  if (!h) { if (error) *error = "libnvidia-ml.so.1 not found"; return out; }
  auto init = sym<int (*)()>(h, "nvmlInit_v2");
  auto shutdown = sym<int (*)()>(h, "nvmlShutdown");
  auto count = sym<int (*)(unsigned*)>(h, "nvmlDeviceGetCount_v2");
  auto handle = sym<int (*)(unsigned, nvmlDevice_t*)>(h, "nvmlDeviceGetHandleByIndex_v2");
  auto name = sym<int (*)(nvmlDevice_t, char*, unsigned)>(h, "nvmlDeviceGetName");
  auto uuid = sym<int (*)(nvmlDevice_t, char*, unsigned)>(h, "nvmlDeviceGetUUID");
  auto mem = sym<int (*)(nvmlDevice_t, nvmlMemory_t*)>(h, "nvmlDeviceGetMemoryInfo");
  auto power = sym<int (*)(nvmlDevice_t, unsigned*)>(h, "nvmlDeviceGetPowerUsage");
  auto temp = sym<int (*)(nvmlDevice_t, int, unsigned*)>(h, "nvmlDeviceGetTemperature");
  auto util = sym<int (*)(nvmlDevice_t, nvmlUtilization_t*)>(h, "nvmlDeviceGetUtilizationRates");
  auto clock = sym<int (*)(nvmlDevice_t, int, unsigned*)>(h, "nvmlDeviceGetClockInfo");
  auto link_state = sym<int (*)(nvmlDevice_t, unsigned, int*)>(h, "nvmlDeviceGetNvLinkState");
  auto link_pci = sym<int (*)(nvmlDevice_t, unsigned, nvmlPciInfo_t*)>(h, "nvmlDeviceGetNvLinkRemotePciInfo_v2");
  auto pci = sym<int (*)(nvmlDevice_t, nvmlPciInfo_t*)>(h, "nvmlDeviceGetPciInfo_v3");
  auto p2p = sym<int (*)(nvmlDevice_t, nvmlDevice_t, int, int*)>(h, "nvmlDeviceGetP2PStatus");
  if (!init || !count || !handle || init() != 0) {
    if (error) *error = "nvmlInit failed";
    dlclose(h);
    return out;
  }
  unsigned n = 0;
  count(&n);
  std::vector<nvmlDevice_t> devs(n);
  std::vector<std::string> bus(n);
  for (unsigned i = 0; i < n; i++) {
    GpuInfo g;
    g.index = (int)i;
    if (handle(i, &devs[i]) != 0) continue;
    char buf[96];
    if (name && name(devs[i], buf, sizeof buf) == 0) g.name = buf;
    if (uuid && uuid(devs[i], buf, sizeof buf) == 0) g.uuid = buf;
    nvmlMemory_t m{};
    if (mem && mem(devs[i], &m) == 0) { g.mem_total = m.total; g.mem_free = m.free; }
    if (power) power(devs[i], &g.power_mw);
    if (temp) temp(devs[i], 0 /* GPU sensor */, &g.temp_c);
    nvmlUtilization_t u{};
    if (util && util(devs[i], &u) == 0) g.util_pct = u.gpu;
    if (clock) clock(devs[i], 1 /* SM */, &g.sm_mhz);
    nvmlPciInfo_t pi{};
    if (pci && pci(devs[i], &pi) == 0) bus[i] = pi.busId;
    out.push_back(g);
  }
  for (auto& g : out) {
    g.nvlink_peers_links.assign(n, 0);
    g.p2p_ok.assign(n, 0);
    for (unsigned l = 0; l < NVML_LINKS && link_state; l++) {
      int active = 0;
      if (link_state(devs[g.index], l, &active) != 0 || !active) continue;
      g.active_links++;
      nvmlPciInfo_t rp{};
      if (link_pci && link_pci(devs[g.index], l, &rp) == 0)
        for (unsigned j = 0; j < n; j++)
          if (j != (unsigned)g.index && bus[j] == rp.busId) g.nvlink_peers_links[j]++;  // direct link (no switch)
    }
    for (unsigned j = 0; j < n && p2p; j++) {
      if (j == (unsigned)g.index) continue;
      int st = -1;
      // index 2 = NVLINK capability; 0 means OK
      if (p2p(devs[g.index], devs[j], 2, &st) == 0 && st == 0) g.p2p_ok[j] = 1;
    }
  }
  if (shutdown) shutdown();
  dlclose(h);
  return out;
}

}  // namespace exo
