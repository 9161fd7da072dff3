// TCP pub/sub bus with liveliness and UDP multicast discovery (see bus.h).
#include "bus.h"

#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <net/if.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <string.h>
#include <sys/epoll.h>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <time.h>
#include <unistd.h>

#include <algorithm>
#include <random>
#include <stdexcept>

namespace exo {

namespace {
constexpr uint32_t FRAME_MAGIC = 0x45584F42;  // "EXOB"
enum FrameKind : uint8_t { F_HELLO = 1, F_SUB = 2, F_UNSUB = 3, F_MSG = 4, F_PING = 5 };
constexpr int64_t PING_MS = 1000, DEAD_MS = 5000, DISC_MS = 1000;
constexpr size_t MAX_FRAME = 64u << 20;

int64_t now_ms() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (int64_t)ts.tv_sec * 1000 + ts.tv_nsec / 1000000;
}
void set_nonblock(int fd, bool on) {
  int fl = fcntl(fd, F_GETFL, 0);
  fcntl(fd, F_SETFL, on ? (fl | O_NONBLOCK) : (fl & ~O_NONBLOCK));
}
bool write_all(int fd, const char* p, size_t n) {
  while (n) {
    ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
    if (w < 0) {
      if (errno == EINTR) continue;
      if (errno == EAGAIN || errno == EWOULDBLOCK) {  // back-pressure: wait for the peer to drain
        pollfd pf{fd, POLLOUT, 0};
        if (::poll(&pf, 1, 5000) <= 0) return false;
        continue;
      }
      return false;
    }
    p += w;
    n -= (size_t)w;
  }
  return true;
}
void put_u16(std::string& s, uint16_t v) { s.push_back((char)(v & 0xff)); s.push_back((char)(v >> 8)); }
void put_u32(std::string& s, uint32_t v) { for (int i = 0; i < 4; i++) s.push_back((char)((v >> (8 * i)) & 0xff)); }
uint32_t get_u32(const char* p) { uint32_t v = 0; for (int i = 0; i < 4; i++) v |= (uint32_t)(uint8_t)p[i] << (8 * i); return v; }
uint16_t get_u16(const char* p) { return (uint16_t)((uint8_t)p[0] | ((uint8_t)p[1] << 8)); }
}  // namespace

uint64_t namespace_hash(const std::string& ns) {
  uint64_t h = 1469598103934665603ull;
  for (unsigned char c : ns) { h ^= c; h *= 1099511628211ull; }
  return h;
}

bool valid_identity(const std::string& id) {
  if (id.empty() || id.size() > 32 || id[0] == '0') return false;
  for (char c : id)
    if (!isxdigit((unsigned char)c)) return false;
  return true;
}

Bus::Bus(const std::string& identity, const std::string& ns, int listen_port, int discovery_port)
    : id_(identity), ns_(namespace_hash(ns)), discovery_port_(discovery_port) {
  if (!valid_identity(identity)) throw std::invalid_argument("identity must be hex, <= 32 digits, no leading zero");
  listen_fd_ = ::socket(AF_INET6, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (listen_fd_ < 0) throw std::runtime_error("socket() failed");
  int zero = 0, one = 1;
  setsockopt(listen_fd_, IPPROTO_IPV6, IPV6_V6ONLY, &zero, sizeof zero);  // dual stack
  setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in6 a{};
  a.sin6_family = AF_INET6;
  a.sin6_addr = in6addr_any;
  a.sin6_port = htons((uint16_t)listen_port);
  if (::bind(listen_fd_, (sockaddr*)&a, sizeof a) < 0 || ::listen(listen_fd_, 64) < 0) {
    ::close(listen_fd_);
    throw std::runtime_error(std::string("bind/listen failed: ") + strerror(errno));
  }
  socklen_t al = sizeof a;
  getsockname(listen_fd_, (sockaddr*)&a, &al);
  listen_port_ = ntohs(a.sin6_port);
  set_nonblock(listen_fd_, true);
  epoll_fd_ = epoll_create1(EPOLL_CLOEXEC);
  event_fd_ = eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC | EFD_SEMAPHORE);
  wake_fd_ = eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
  epoll_event ev{};
  ev.events = EPOLLIN;
  ev.data.fd = listen_fd_;
  epoll_ctl(epoll_fd_, EPOLL_CTL_ADD, listen_fd_, &ev);
  ev.data.fd = wake_fd_;
  epoll_ctl(epoll_fd_, EPOLL_CTL_ADD, wake_fd_, &ev);
  if (discovery_port_ > 0) {
    disc_fd_ = ::socket(AF_INET6, SOCK_DGRAM | SOCK_CLOEXEC | SOCK_NONBLOCK, 0);
    if (disc_fd_ >= 0) {
      setsockopt(disc_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
#ifdef SO_REUSEPORT
      setsockopt(disc_fd_, SOL_SOCKET, SO_REUSEPORT, &one, sizeof one);
#endif
      sockaddr_in6 d{};
      d.sin6_family = AF_INET6;
      d.sin6_addr = in6addr_any;
      d.sin6_port = htons((uint16_t)discovery_port_);
      if (::bind(disc_fd_, (sockaddr*)&d, sizeof d) == 0) {
        ipv6_mreq mr{};
        inet_pton(AF_INET6, DISC_GROUP, &mr.ipv6mr_multiaddr);
        if (struct if_nameindex* ifs = if_nameindex()) {   // join on every interface; failures are fine
          for (auto* i = ifs; i->if_index; i++) {
            mr.ipv6mr_interface = i->if_index;
            setsockopt(disc_fd_, IPPROTO_IPV6, IPV6_JOIN_GROUP, &mr, sizeof mr);
          }
          if_freenameindex(ifs);
        }
        ev.data.fd = disc_fd_;
        epoll_ctl(epoll_fd_, EPOLL_CTL_ADD, disc_fd_, &ev);
      } else {
        ::close(disc_fd_);
        disc_fd_ = -1;
      }
    }
  }
  io_ = std::thread([this] { io_loop(); });
}

Bus::~Bus() { close(); }

void Bus::close() {
  if (stop_.exchange(true)) return;
  uint64_t one = 1;
  (void)!::write(wake_fd_, &one, sizeof one);
  if (io_.joinable()) io_.join();
  std::lock_guard<std::mutex> lk(mu_);
  for (auto& kv : peers_) ::close(kv.first);
  peers_.clear();
  for (int* fd : {&listen_fd_, &epoll_fd_, &wake_fd_, &disc_fd_}) {
    if (*fd >= 0) ::close(*fd);
    *fd = -1;
  }
  // event_fd_ stays open until destruction of the Python wrapper reads the last events
}

void Bus::push_event(BusEvent&& e) {
  {
    std::lock_guard<std::mutex> lk(mu_);
    events_.push_back(std::move(e));
  }
  uint64_t one = 1;
  (void)!::write(event_fd_, &one, sizeof one);
}

bool Bus::try_recv(BusEvent* out) {
  std::lock_guard<std::mutex> lk(mu_);
  if (events_.empty()) return false;
  *out = std::move(events_.front());
  events_.pop_front();
  uint64_t v;
  (void)!::read(event_fd_, &v, sizeof v);  // semaphore mode: one count per event
  return true;
}

bool Bus::send_frame(const std::shared_ptr<Peer>& p, uint8_t kind, const std::string& topic, const std::string& data) {
  std::string f;
  f.reserve(16 + topic.size() + data.size());
  put_u32(f, FRAME_MAGIC);
  f.push_back((char)kind);
  put_u16(f, (uint16_t)topic.size());
  put_u32(f, (uint32_t)data.size());
  f += topic;
  f += data;
  std::lock_guard<std::mutex> lk(p->wmu);
  return p->fd >= 0 && write_all(p->fd, f.data(), f.size());
}

void Bus::add_peer_fd(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
  int buf = 16 << 20;
  setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &buf, sizeof buf);
  set_nonblock(fd, true);
  auto p = std::make_shared<Peer>();
  p->fd = fd;
  p->last_seen_ms = now_ms();
  std::vector<std::string> subs;
  {
    std::lock_guard<std::mutex> lk(mu_);
    peers_[fd] = p;
    subs.assign(subs_.begin(), subs_.end());
  }
  std::string hello = id_;
  hello.append((const char*)&ns_, sizeof ns_);
  send_frame(p, F_HELLO, "", hello);
  for (auto& t : subs) send_frame(p, F_SUB, t, "");
  epoll_event ev{};
  ev.events = EPOLLIN | EPOLLRDHUP;
  ev.data.fd = fd;
  epoll_ctl(epoll_fd_, EPOLL_CTL_ADD, fd, &ev);
}

bool Bus::connect_to(const std::string& host, int port) {
  addrinfo hints{}, *res = nullptr;
  hints.ai_socktype = SOCK_STREAM;
  if (getaddrinfo(host.c_str(), std::to_string(port).c_str(), &hints, &res) != 0) return false;
  int fd = -1;
  for (auto* ai = res; ai; ai = ai->ai_next) {
    fd = ::socket(ai->ai_family, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) continue;
    if (::connect(fd, ai->ai_addr, ai->ai_addrlen) == 0) break;
    ::close(fd);
    fd = -1;
  }
  freeaddrinfo(res);
  if (fd < 0) return false;
  add_peer_fd(fd);
  return true;
}

void Bus::accept_new() {
  for (;;) {
    int fd = ::accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
    if (fd < 0) return;
    add_peer_fd(fd);
  }
}

void Bus::drop_peer(const std::shared_ptr<Peer>& p) {
  bool announce = false;
  std::string id;
  {
    std::lock_guard<std::mutex> lk(mu_);
    if (peers_.erase(p->fd) == 0) return;
    announce = p->announced;
    id = p->id;
  }
  epoll_ctl(epoll_fd_, EPOLL_CTL_DEL, p->fd, nullptr);
  {
    std::lock_guard<std::mutex> lk(p->wmu);
    ::close(p->fd);
    p->fd = -1;
  }
  if (announce) {
    BusEvent e;
    e.kind = BusEvent::Connection;
    e.peer = id;
    e.connected = false;
    push_event(std::move(e));
  }
}

bool Bus::parse_frames(const std::shared_ptr<Peer>& p) {
  std::string& b = p->inbuf;
  size_t off = 0;
  while (b.size() - off >= 11) {
    const char* h = b.data() + off;
    if (get_u32(h) != FRAME_MAGIC) return false;
    uint8_t kind = (uint8_t)h[4];
    size_t tl = get_u16(h + 5), dl = get_u32(h + 7);
    if (dl > MAX_FRAME) return false;
    if (b.size() - off < 11 + tl + dl) break;
    std::string topic(h + 11, tl), data(h + 11 + tl, dl);
    off += 11 + tl + dl;
    switch (kind) {
      case F_HELLO: {
        if (data.size() < sizeof(uint64_t) + 1) return false;
        uint64_t ns;
        memcpy(&ns, data.data() + data.size() - sizeof ns, sizeof ns);
        if (ns != ns_) return false;  // another cluster: hang up
        std::string id = data.substr(0, data.size() - sizeof ns);
        if (id == id_) return false;  // ourselves
        bool dup = false;
        {
          std::lock_guard<std::mutex> lk(mu_);
          for (auto& kv : peers_) dup |= (kv.second != p && kv.second->id == id);
          if (!dup) { p->id = id; p->announced = true; }
        }
        if (dup) return false;        // one connection per peer pair
        BusEvent e;
        e.kind = BusEvent::Connection;
        e.peer = id;
        e.connected = true;
        push_event(std::move(e));
        break;
      }
      case F_SUB: { std::lock_guard<std::mutex> lk(mu_); p->subs.insert(topic); break; }
      case F_UNSUB: { std::lock_guard<std::mutex> lk(mu_); p->subs.erase(topic); break; }
      case F_MSG: {
        bool want;
        { std::lock_guard<std::mutex> lk(mu_); want = subs_.count(topic) > 0; }
        if (want) {
          BusEvent e;
          e.kind = BusEvent::Message;
          e.peer = p->id;
          e.topic = std::move(topic);
          e.data = std::move(data);
          push_event(std::move(e));
        }
        break;
      }
      case F_PING: break;
      default: return false;
    }
  }
  b.erase(0, off);
  return true;
}

void Bus::on_readable(const std::shared_ptr<Peer>& p) {
  char buf[65536];
  for (;;) {
    ssize_t n = ::recv(p->fd, buf, sizeof buf, 0);
    if (n > 0) {
      p->inbuf.append(buf, (size_t)n);
      p->last_seen_ms = now_ms();
      continue;
    }
    if (n == 0) { drop_peer(p); return; }
    if (errno == EINTR) continue;
    if (errno == EAGAIN || errno == EWOULDBLOCK) break;
    drop_peer(p);
    return;
  }
  if (!parse_frames(p)) drop_peer(p);
}

void Bus::subscribe(const std::string& topic) {
  std::vector<std::shared_ptr<Peer>> ps;
  {
    std::lock_guard<std::mutex> lk(mu_);
    if (!subs_.insert(topic).second) return;
    for (auto& kv : peers_) ps.push_back(kv.second);
  }
  for (auto& p : ps) send_frame(p, F_SUB, topic, "");
}

void Bus::unsubscribe(const std::string& topic) {
  std::vector<std::shared_ptr<Peer>> ps;
  {
    std::lock_guard<std::mutex> lk(mu_);
    if (!subs_.erase(topic)) return;
    for (auto& kv : peers_) ps.push_back(kv.second);
  }
  for (auto& p : ps) send_frame(p, F_UNSUB, topic, "");
}

int Bus::publish(const std::string& topic, const std::string& data) {
  std::vector<std::shared_ptr<Peer>> ps;
  {
    std::lock_guard<std::mutex> lk(mu_);
    for (auto& kv : peers_)
      if (kv.second->announced && kv.second->subs.count(topic)) ps.push_back(kv.second);
  }
  int n = 0;
  for (auto& p : ps) n += send_frame(p, F_MSG, topic, data) ? 1 : 0;
  return n;
}

std::vector<std::string> Bus::peers() {
  std::vector<std::string> out;
  std::lock_guard<std::mutex> lk(mu_);
  for (auto& kv : peers_)
    if (kv.second->announced) out.push_back(kv.second->id);
  return out;
}

// ---- discovery -----------------------------------------------------------------------------------
void Bus::discovery_tick() {
  if (disc_fd_ < 0) return;
  static thread_local std::mt19937_64 rng{std::random_device{}()};
  uint64_t r = rng();
  memcpy(last_nonce_, &r, 8);
  DiscHello m{};
  memcpy(m.h.magic, "EXO", 3);
  m.h.kind = DISC_HELLO;
  memcpy(m.nonce, last_nonce_, 8);
  memcpy(m.ns, &ns_, 8);
  sockaddr_in6 to{};
  to.sin6_family = AF_INET6;
  to.sin6_port = htons((uint16_t)discovery_port_);
  inet_pton(AF_INET6, DISC_GROUP, &to.sin6_addr);
  if (struct if_nameindex* ifs = if_nameindex()) {
    for (auto* i = ifs; i->if_index; i++) {
      to.sin6_scope_id = i->if_index;
      unsigned idx = i->if_index;
      setsockopt(disc_fd_, IPPROTO_IPV6, IPV6_MULTICAST_IF, &idx, sizeof idx);
      ::sendto(disc_fd_, &m, sizeof m, 0, (sockaddr*)&to, sizeof to);
    }
    if_freenameindex(ifs);
  }
}

void Bus::on_discovery_packet() {
  for (;;) {
    uint8_t buf[64];
    sockaddr_in6 from{};
    socklen_t fl = sizeof from;
    ssize_t n = ::recvfrom(disc_fd_, buf, sizeof buf, 0, (sockaddr*)&from, &fl);
    if (n < (ssize_t)sizeof(DiscHeader)) return;
    auto* h = (DiscHeader*)buf;
    if (memcmp(h->magic, "EXO", 3) != 0) continue;
    if (h->kind == DISC_HELLO && n >= (ssize_t)sizeof(DiscHello)) {
      auto* m = (DiscHello*)buf;
      if (memcmp(m->ns, &ns_, 8) != 0 || memcmp(m->nonce, last_nonce_, 8) == 0) continue;  // other cluster / our own echo
      DiscWhatsUp w{};
      memcpy(w.h.magic, "EXO", 3);
      w.h.kind = DISC_WHATSUP;
      memcpy(w.nonce, m->nonce, 8);
      memset(w.id, 0, 16);
      // identity is up to 32 hex digits = 16 bytes, right-aligned
      std::string hex = std::string(32 - id_.size(), '0') + id_;
      for (int i = 0; i < 16; i++) w.id[i] = (uint8_t)strtoul(hex.substr(2 * i, 2).c_str(), nullptr, 16);
      w.port_le[0] = (uint8_t)(listen_port_ & 0xff);
      w.port_le[1] = (uint8_t)(listen_port_ >> 8);
      ::sendto(disc_fd_, &w, sizeof w, 0, (sockaddr*)&from, fl);
    } else if (h->kind == DISC_WHATSUP && n >= (ssize_t)sizeof(DiscWhatsUp)) {
      auto* w = (DiscWhatsUp*)buf;
      if (memcmp(w->nonce, last_nonce_, 8) != 0) continue;
      char hex[33];
      for (int i = 0; i < 16; i++) snprintf(hex + 2 * i, 3, "%02x", w->id[i]);
      std::string id(hex);
      id.erase(0, std::min(id.find_first_not_of('0'), id.size() - 1));
      if (id == id_) continue;
      char addr[INET6_ADDRSTRLEN];
      inet_ntop(AF_INET6, &from.sin6_addr, addr, sizeof addr);
      int port = w->port_le[0] | (w->port_le[1] << 8);
      std::string host = addr;
      if (IN6_IS_ADDR_LINKLOCAL(&from.sin6_addr)) {
        char ifn[IF_NAMESIZE];
        if (if_indextoname(from.sin6_scope_id, ifn)) host += std::string("%") + ifn;
      }
      BusEvent e;
      e.kind = BusEvent::Discovered;
      e.peer = id;
      e.data = host + ":" + std::to_string(port);
      push_event(std::move(e));
      // the reference rule: the side whose id is not smaller opens the connection
      bool known;
      { std::lock_guard<std::mutex> lk(mu_); known = false; for (auto& kv : peers_) known |= kv.second->id == id; }
      if (!known && id_ >= id) connect_to(host, port);
    }
  }
}

void Bus::io_loop() {
  int64_t next_ping = now_ms() + PING_MS, next_disc = now_ms();
  while (!stop_) {
    epoll_event evs[32];
    int n = epoll_wait(epoll_fd_, evs, 32, 200);
    for (int i = 0; i < n && !stop_; i++) {
      int fd = evs[i].data.fd;
      if (fd == listen_fd_) { accept_new(); continue; }
      if (fd == wake_fd_) { uint64_t v; (void)!::read(wake_fd_, &v, sizeof v); continue; }
      if (fd == disc_fd_) { on_discovery_packet(); continue; }
      std::shared_ptr<Peer> p;
      { std::lock_guard<std::mutex> lk(mu_); auto it = peers_.find(fd); if (it != peers_.end()) p = it->second; }
      if (!p) continue;
      if (evs[i].events & (EPOLLHUP | EPOLLERR)) { drop_peer(p); continue; }
      on_readable(p);
      if (evs[i].events & EPOLLRDHUP) drop_peer(p);
    }
    int64_t t = now_ms();
    if (t >= next_ping) {
      next_ping = t + PING_MS;
      std::vector<std::shared_ptr<Peer>> ps;
      { std::lock_guard<std::mutex> lk(mu_); for (auto& kv : peers_) ps.push_back(kv.second); }
      for (auto& p : ps) {
        if (t - p->last_seen_ms > DEAD_MS) drop_peer(p);
        else send_frame(p, F_PING, "", "");
      }
    }
    if (disc_fd_ >= 0 && t >= next_disc) { next_disc = t + DISC_MS; discovery_tick(); }
  }
}

}  // namespace exo
