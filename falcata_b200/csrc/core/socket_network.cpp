// Host collectives over TCP for multi-process training on CPUs (the command line's distributed mode, FB_NetworkInit).
//
// Every process listens on its own port and the processes form a full mesh: a process connects to every entry that
// precedes it in the machine list and accepts a connection from every entry that follows it; the first word on a new
// connection is the connecting side's rank. Two collectives are installed into fb::Network, the same two that an
// embedding process may inject: an all-gather (ring of pairwise exchanges: in step s a rank sends its block to rank + s
// and receives the block of rank - s, both directions driven by one poll loop so that large blocks cannot deadlock on
// full socket buffers) and a sum all-reduce built on it (every rank adds the gathered blocks in rank order, so all
// ranks hold bit-identical sums). Histograms of the host learner are a few hundred kilobytes, so the all-gather form
// costs little against the local work. The histogram exchange of the data-parallel learner uses the third collective, a
// reduce-scatter with per-rank block sizes: a rank sends every peer only the bins of the features that peer searches and
// sums what it receives for its own features in rank order (the same sums as the all-reduce gives).
//
// Parity: src/network/linkers_socket.cpp:L26-222 (listen / connect mesh from the machine list), src/network/network.cpp
// (Allreduce / Allgather), include/Falcata/c_api.h FLC_NetworkInit.
#include "fb/learner.h"

#include <arpa/inet.h>
#include <fcntl.h>
#include <ifaddrs.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <chrono>
#include <cstring>
#include <fstream>
#include <sstream>
#include <thread>

namespace fb {

namespace {

struct Mesh {
  int rank = 0, world = 1, listen_fd = -1;
  std::vector<int> fd;   // fd[r]: connection to rank r (-1 for this rank)
  int op_timeout_ms = 600000;   // a collective without progress for this long ends with an error (time_out, in minutes, at init)
  bool up = false;
};
Mesh g_mesh;

struct Endpoint { std::string host; int port = 0; };

void CloseMesh() {
  for (int f : g_mesh.fd) if (f >= 0) close(f);
  if (g_mesh.listen_fd >= 0) close(g_mesh.listen_fd);
  g_mesh = Mesh();
}

void SendAll(int fd, const char* p, size_t n) {
  while (n > 0) {
    const ssize_t k = send(fd, p, n, MSG_NOSIGNAL);
    if (k < 0) { if (errno == EINTR) continue; Log::Fatal("Socket send failed: %s", strerror(errno)); }
    p += k; n -= static_cast<size_t>(k);
  }
}

void RecvAll(int fd, char* p, size_t n) {
  while (n > 0) {
    const ssize_t k = recv(fd, p, n, 0);
    if (k == 0) Log::Fatal("A peer closed its connection (another machine stopped)");
    if (k < 0) { if (errno == EINTR) continue; Log::Fatal("Socket receive failed: %s", strerror(errno)); }
    p += k; n -= static_cast<size_t>(k);
  }
}

// Sends sn bytes on fd_s while receiving rn bytes on fd_r (the two may be the same connection). Neither direction waits
// for the other: both are advanced whenever the kernel can take or give bytes.
void SendRecv(int fd_s, const char* sp, size_t sn, int fd_r, char* rp, size_t rn) {
  while (sn > 0 || rn > 0) {
    pollfd p[2]; int np = 0, is = -1, ir = -1;
    if (fd_s == fd_r) { p[0].fd = fd_s; p[0].events = static_cast<short>((sn > 0 ? POLLOUT : 0) | (rn > 0 ? POLLIN : 0)); p[0].revents = 0; is = ir = 0; np = 1; }
    else {
      if (sn > 0) { p[np].fd = fd_s; p[np].events = POLLOUT; p[np].revents = 0; is = np++; }
      if (rn > 0) { p[np].fd = fd_r; p[np].events = POLLIN; p[np].revents = 0; ir = np++; }
    }
    const int rc = poll(p, np, g_mesh.op_timeout_ms);
    if (rc < 0) { if (errno == EINTR) continue; Log::Fatal("poll failed: %s", strerror(errno)); }
    if (rc == 0) Log::Fatal("No progress on a collective for %d s (time_out): a peer machine is not taking part", g_mesh.op_timeout_ms / 1000);
    if (sn > 0 && is >= 0 && (p[is].revents & (POLLOUT | POLLERR | POLLHUP))) {
      const ssize_t k = send(fd_s, sp, sn, MSG_NOSIGNAL | MSG_DONTWAIT);
      if (k < 0) { if (errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) Log::Fatal("Socket send failed: %s", strerror(errno)); }
      else { sp += k; sn -= static_cast<size_t>(k); }
    }
    if (rn > 0 && ir >= 0 && (p[ir].revents & (POLLIN | POLLERR | POLLHUP))) {
      const ssize_t k = recv(fd_r, rp, rn, MSG_DONTWAIT);
      if (k == 0) Log::Fatal("A peer closed its connection (another machine stopped)");
      if (k < 0) { if (errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) Log::Fatal("Socket receive failed: %s", strerror(errno)); }
      else { rp += k; rn -= static_cast<size_t>(k); }
    }
  }
}

void MeshAllgather(const void* in, int64_t bytes, void* out) {
  char* o = static_cast<char*>(out);
  const size_t b = static_cast<size_t>(bytes);
  if (o + static_cast<size_t>(g_mesh.rank) * b != in) memcpy(o + static_cast<size_t>(g_mesh.rank) * b, in, b);
  for (int s = 1; s < g_mesh.world; ++s) {
    const int to = (g_mesh.rank + s) % g_mesh.world, from = (g_mesh.rank - s + g_mesh.world) % g_mesh.world;
    SendRecv(g_mesh.fd[to], static_cast<const char*>(in), b, g_mesh.fd[from], o + static_cast<size_t>(from) * b, b);
  }
}

void MeshAllreduceSum(void* buf, int64_t count, int dtype) {
  const size_t bytes = static_cast<size_t>(count) * 8;
  std::vector<char> all(bytes * g_mesh.world);
  MeshAllgather(buf, static_cast<int64_t>(bytes), all.data());
  if (dtype == 0) {
    double* d = static_cast<double*>(buf);
    for (int64_t i = 0; i < count; ++i) { double s = 0.0; for (int r = 0; r < g_mesh.world; ++r) s += reinterpret_cast<const double*>(all.data() + r * bytes)[i]; d[i] = s; }
  } else {
    int64_t* d = static_cast<int64_t*>(buf);
    for (int64_t i = 0; i < count; ++i) { int64_t s = 0; for (int r = 0; r < g_mesh.world; ++r) s += reinterpret_cast<const int64_t*>(all.data() + r * bytes)[i]; d[i] = s; }
  }
}

void MeshReduceScatter(const void* sendbuf, const int64_t* counts, void* recv, int dtype) {
  const int W = g_mesh.world, R = g_mesh.rank;
  const size_t mine = static_cast<size_t>(counts[R]) * 8;
  std::vector<size_t> start(W + 1, 0);
  for (int r = 0; r < W; ++r) start[r + 1] = start[r] + static_cast<size_t>(counts[r]) * 8;
  const char* send = static_cast<const char*>(sendbuf);
  std::vector<char> stage(mine * W);                       // [source rank][own block]
  memcpy(stage.data() + static_cast<size_t>(R) * mine, send + start[R], mine);
  for (int s = 1; s < W; ++s) {
    const int to = (R + s) % W, from = (R - s + W) % W;
    SendRecv(g_mesh.fd[to], send + start[to], start[to + 1] - start[to], g_mesh.fd[from], stage.data() + static_cast<size_t>(from) * mine, mine);
  }
  const int64_t n = counts[R];
  if (dtype == 0) {
    double* d = static_cast<double*>(recv);
    for (int64_t i = 0; i < n; ++i) { double a = 0.0; for (int r = 0; r < W; ++r) a += reinterpret_cast<const double*>(stage.data() + static_cast<size_t>(r) * mine)[i]; d[i] = a; }
  } else {
    int64_t* d = static_cast<int64_t*>(recv);
    for (int64_t i = 0; i < n; ++i) { int64_t a = 0; for (int r = 0; r < W; ++r) a += reinterpret_cast<const int64_t*>(stage.data() + static_cast<size_t>(r) * mine)[i]; d[i] = a; }
  }
}

bool IsLocalAddress(const std::string& host) {
  if (host == "127.0.0.1" || host == "localhost" || host == "0.0.0.0" || host == "::1") return true;
  ifaddrs* list = nullptr;
  if (getifaddrs(&list) != 0) return false;
  bool found = false;
  for (ifaddrs* a = list; a != nullptr && !found; a = a->ifa_next) {
    if (a->ifa_addr == nullptr || a->ifa_addr->sa_family != AF_INET) continue;
    char buf[INET_ADDRSTRLEN];
    if (inet_ntop(AF_INET, &reinterpret_cast<sockaddr_in*>(a->ifa_addr)->sin_addr, buf, sizeof(buf)) != nullptr && host == buf) found = true;
  }
  freeifaddrs(list);
  if (!found) { char name[256]; if (gethostname(name, sizeof(name)) == 0 && host == name) found = true; }
  return found;
}

std::vector<Endpoint> ParseMachines(const std::string& machines) {
  // "host:port,host:port" or lines of "host port" (a machine list file's content)
  std::vector<Endpoint> out;
  std::string text = machines;
  for (char& c : text) if (c == ',' || c == '\n' || c == '\r' || c == ';') c = '\n';
  std::stringstream ss(text); std::string line;
  while (std::getline(ss, line)) {
    line = Trim(line);
    if (line.empty() || line[0] == '#') continue;
    size_t sep = line.find_last_of(": \t");
    if (sep == std::string::npos) Log::Fatal("Machine list entry \"%s\" has no port (write host:port or \"host port\")", line.c_str());
    Endpoint e; e.host = Trim(line.substr(0, sep)); e.port = atoi(line.substr(sep + 1).c_str());
    if (e.host.empty() || e.port <= 0) Log::Fatal("Machine list entry \"%s\" is not host:port", line.c_str());
    out.push_back(e);
  }
  return out;
}

int ConnectTo(const Endpoint& e, std::chrono::steady_clock::time_point deadline) {
  addrinfo hints; memset(&hints, 0, sizeof(hints)); hints.ai_family = AF_INET; hints.ai_socktype = SOCK_STREAM;
  for (;;) {
    addrinfo* res = nullptr;
    if (getaddrinfo(e.host.c_str(), std::to_string(e.port).c_str(), &hints, &res) == 0 && res != nullptr) {
      const int fd = socket(res->ai_family, res->ai_socktype, res->ai_protocol);
      if (fd >= 0) {
        if (connect(fd, res->ai_addr, res->ai_addrlen) == 0) { freeaddrinfo(res); return fd; }
        close(fd);
      }
      freeaddrinfo(res);
    }
    if (std::chrono::steady_clock::now() > deadline) Log::Fatal("Cannot connect to %s:%d within the time limit (is that machine's process running?)", e.host.c_str(), e.port);
    std::this_thread::sleep_for(std::chrono::milliseconds(100));
  }
}

}  // namespace

// Joins the mesh described by `machines` as the process that listens on local_listen_port. `timeout_minutes` bounds the
// wait for the other processes to come up. Installs the collectives into fb::Network.
void SocketNetworkInit(const std::string& machines, int local_listen_port, int timeout_minutes, int num_machines) {
  CloseMesh();
  std::vector<Endpoint> list = ParseMachines(machines);
  if (num_machines > 0 && static_cast<int>(list.size()) > num_machines) list.resize(num_machines);
  if (static_cast<int>(list.size()) < std::max(2, num_machines)) Log::Fatal("The machine list has %d entries; num_machines=%d needs as many (at least 2)", static_cast<int>(list.size()), num_machines);
  const int world = static_cast<int>(list.size());
  int rank = -1;
  for (int r = 0; r < world; ++r) if (list[r].port == local_listen_port && IsLocalAddress(list[r].host)) { rank = r; break; }
  if (rank < 0) Log::Fatal("No entry of the machine list is this machine on port %d (local_listen_port)", local_listen_port);
  g_mesh.rank = rank; g_mesh.world = world; g_mesh.fd.assign(world, -1);
  g_mesh.op_timeout_ms = static_cast<int>(std::min<long long>(static_cast<long long>(std::max(1, timeout_minutes)) * 60000LL, 1LL << 30));

  g_mesh.listen_fd = socket(AF_INET, SOCK_STREAM, 0);
  if (g_mesh.listen_fd < 0) Log::Fatal("Cannot create a socket: %s", strerror(errno));
  int one = 1; setsockopt(g_mesh.listen_fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in addr; memset(&addr, 0, sizeof(addr)); addr.sin_family = AF_INET; addr.sin_addr.s_addr = htonl(INADDR_ANY); addr.sin_port = htons(static_cast<uint16_t>(local_listen_port));
  if (bind(g_mesh.listen_fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0) Log::Fatal("Cannot bind port %d: %s", local_listen_port, strerror(errno));
  if (listen(g_mesh.listen_fd, world) != 0) Log::Fatal("Cannot listen on port %d: %s", local_listen_port, strerror(errno));

  const auto deadline = std::chrono::steady_clock::now() + std::chrono::minutes(std::max(1, timeout_minutes));
  for (int r = 0; r < rank; ++r) {
    const int fd = ConnectTo(list[r], deadline);
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    const int32_t me = rank; SendAll(fd, reinterpret_cast<const char*>(&me), sizeof(me));
    g_mesh.fd[r] = fd;
  }
  for (int pending = world - 1 - rank; pending > 0; --pending) {
    pollfd p; p.fd = g_mesh.listen_fd; p.events = POLLIN; p.revents = 0;
    const auto left = std::chrono::duration_cast<std::chrono::milliseconds>(deadline - std::chrono::steady_clock::now()).count();
    if (left <= 0 || poll(&p, 1, static_cast<int>(std::min<long long>(left, 1 << 30))) <= 0) Log::Fatal("Timed out waiting for %d more machine(s) to connect to port %d", pending, local_listen_port);
    const int fd = accept(g_mesh.listen_fd, nullptr, nullptr);
    if (fd < 0) Log::Fatal("accept failed: %s", strerror(errno));
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    int32_t peer = -1; RecvAll(fd, reinterpret_cast<char*>(&peer), sizeof(peer));
    if (peer <= rank || peer >= world || g_mesh.fd[peer] >= 0) Log::Fatal("Unexpected connection from rank %d", peer);
    g_mesh.fd[peer] = fd;
  }
  g_mesh.up = true;
  Network::world() = world; Network::rank() = rank;
  Network::allreduce() = &MeshAllreduceSum; Network::allgather() = &MeshAllgather; Network::reduce_scatter() = &MeshReduceScatter;
  Log::Info("Connected to %d other machine(s); this is rank %d of %d", world - 1, rank, world);
}

bool SocketNetworkActive() { return g_mesh.up; }

void SocketNetworkFree() {
  if (!g_mesh.up) return;
  Network::world() = 1; Network::rank() = 0; Network::allreduce() = nullptr; Network::allgather() = nullptr; Network::reduce_scatter() = nullptr;
  CloseMesh();
}

void GatherRowCounts(int64_t local_rows, int64_t* global_offset, int64_t* global_total) {
  std::vector<char> raw; Network::Gather(&local_rows, sizeof(local_rows), &raw);
  const int64_t* counts = reinterpret_cast<const int64_t*>(raw.data());
  *global_offset = 0; *global_total = 0;
  for (int r = 0; r < Network::world(); ++r) { if (r == Network::rank()) *global_offset = *global_total; *global_total += counts[r]; }
}

void AllGatherSampleRows(std::vector<double>* sample, int ncol) {
  // sizes first, then the rows padded to the largest sample
  const int W = Network::world();
  int64_t info[2] = {static_cast<int64_t>(sample->size() / std::max(1, ncol)), ncol};
  std::vector<char> raw; Network::Gather(info, sizeof(info), &raw);
  const int64_t* all = reinterpret_cast<const int64_t*>(raw.data());
  int64_t cap = 1;
  for (int r = 0; r < W; ++r) {
    cap = std::max(cap, all[2 * r]);
    if (all[2 * r + 1] != ncol) Log::Fatal("The processes' data have different numbers of columns (%lld against %d)", static_cast<long long>(all[2 * r + 1]), ncol);
  }
  std::vector<double> padded(static_cast<size_t>(cap) * ncol, 0.0); std::copy(sample->begin(), sample->end(), padded.begin());
  std::vector<char> gathered; Network::Gather(padded.data(), static_cast<int64_t>(padded.size() * sizeof(double)), &gathered);
  std::vector<double> merged;
  for (int r = 0; r < W; ++r) {
    const double* p = reinterpret_cast<const double*>(gathered.data()) + static_cast<size_t>(r) * cap * ncol;
    merged.insert(merged.end(), p, p + static_cast<size_t>(all[2 * r]) * ncol);
  }
  sample->swap(merged);
}

// The content of a machine list file ("host port" or "host:port" per line).
std::string ReadMachineListFile(const std::string& path) {
  std::ifstream f(path);
  if (!f) Log::Fatal("Cannot open machine list file %s", path.c_str());
  std::stringstream ss; ss << f.rdbuf();
  return ss.str();
}

}  // namespace fb
