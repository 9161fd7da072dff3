// Node-to-node message bus: topic pub/sub over TCP with peer liveliness and LAN discovery.
//
// Stands where the reference has its Rust `networking` crate on zenoh (session / swarm /
// discovery: rust/networking/src/{lib,swarm,discovery}.rs): a router-mode session that listens on
// a TCP port, connects to discovered peers, publishes to *remote* subscribers only with
// back-pressure (a publish blocks until the frame is handed to every interested peer's socket),
// reports peers coming and going, and isolates clusters by a namespace hash carried in the
// handshake.  Discovery keeps the reference's UDP wire format (magic "EXO", Hello{nonce,namespace},
// WhatsUp{nonce,id,port} on the IPv6 multicast group ff12::e0a1:de89) so packet-level tests and
// tooling carry over; on one box peers can also be given explicitly with connect().
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <thread>
#include <vector>

namespace exo {

// ---- discovery wire format (packed PODs) ---------------------------------------------------
#pragma pack(push, 1)
struct DiscHeader { char magic[3]; uint8_t kind; };           // kind: 1 = Hello, 2 = WhatsUp
struct DiscHello { DiscHeader h; uint8_t nonce[8]; uint8_t ns[8]; };
struct DiscWhatsUp { DiscHeader h; uint8_t nonce[8]; uint8_t id[16]; uint8_t port_le[2]; };
#pragma pack(pop)
constexpr uint8_t DISC_HELLO = 1, DISC_WHATSUP = 2;
constexpr const char* DISC_GROUP = "ff12::e0a1:de89";

// 8-byte namespace tag (FNV-1a 64 of the namespace string; only equality matters)
uint64_t namespace_hash(const std::string& ns);
// Identity rule of the reference: hex, at most 32 digits, no leading zero.
bool valid_identity(const std::string& id);

struct BusEvent {
  enum Kind { Connection = 0, Message = 1, Discovered = 2 } kind;
  std::string peer;      // Connection / Discovered: peer identity
  bool connected = false;
  std::string topic;     // Message
  std::string data;      // Message payload; Discovered: "host:port"
};

class Bus {
 public:
  Bus(const std::string& identity, const std::string& ns, int listen_port, int discovery_port);
  ~Bus();
  int listen_port() const { return listen_port_; }
  int event_fd() const { return event_fd_; }       // readable whenever events are queued
  bool try_recv(BusEvent* out);                    // non-blocking pop
  bool connect_to(const std::string& host, int port);
  void subscribe(const std::string& topic);
  void unsubscribe(const std::string& topic);
  // Blocks until the frame is written to every connected peer subscribed to `topic`.
  // Returns the number of peers it went to.
  int publish(const std::string& topic, const std::string& data);
  std::vector<std::string> peers();
  void close();

 private:
  struct Peer {
    int fd = -1;
    std::string id;            // empty until the handshake arrived
    std::string inbuf;
    std::set<std::string> subs;
    std::mutex wmu;            // serialises writers (publishers and the io thread)
    int64_t last_seen_ms = 0;
    bool announced = false;
  };
  void io_loop();
  void accept_new();
  void on_readable(const std::shared_ptr<Peer>& p);
  bool parse_frames(const std::shared_ptr<Peer>& p);
  void drop_peer(const std::shared_ptr<Peer>& p);
  bool send_frame(const std::shared_ptr<Peer>& p, uint8_t kind, const std::string& topic, const std::string& data);
  void push_event(BusEvent&& e);
  void add_peer_fd(int fd);
  void discovery_tick();
  void on_discovery_packet();

  std::string id_;
  uint64_t ns_;
  int listen_fd_ = -1, listen_port_ = 0, epoll_fd_ = -1, event_fd_ = -1, wake_fd_ = -1, disc_fd_ = -1;
  int discovery_port_ = 0;
  uint8_t last_nonce_[8] = {0};
  std::atomic<bool> stop_{false};
  std::thread io_;
  std::mutex mu_;                                   // peers_, subs_, events_
  std::map<int, std::shared_ptr<Peer>> peers_;
  std::set<std::string> subs_;
  std::deque<BusEvent> events_;
};

// ---- pidfile ---------------------------------------------------------------------------------
// Locked PID file (flock): create + lock, write the pid after daemonising, removed on close.
class Pidfile {
 public:
  explicit Pidfile(const std::string& path);   // throws std::runtime_error("AlreadyRunning:<pid>") if locked
  ~Pidfile();
  void write();
  int raw_fd() const { return fd_; }
  void close();
 private:
  std::string path_;
  int fd_ = -1;
};

// ---- NVML topology ----------------------------------------------------------------------------
struct GpuInfo {
  int index = 0;
  std::string name, uuid;
  uint64_t mem_total = 0, mem_free = 0;
  unsigned power_mw = 0, temp_c = 0, util_pct = 0, sm_mhz = 0;
  std::vector<int> nvlink_peers_links;   // [peer index] -> active NVLink count routed to that peer (0 = none / via switch unknown)
  std::vector<int> p2p_ok;               // [peer index] -> 1 when NVML reports P2P read+write over NVLink
  int active_links = 0;
};
// Empty vector when libnvidia-ml cannot be loaded (no driver): callers fall back to "no GPUs".
std::vector<GpuInfo> nvml_enumerate(std::string* error);

}  // namespace exo
