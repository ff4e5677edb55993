#include "env.h"

#include <arpa/inet.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <netinet/in.h>
#include <sys/socket.h>
#include <unistd.h>

#include <random>
#include <set>

namespace PS {

Options Options::Parse(const std::vector<std::string>& args) {
  Options o;
  auto as_bool = [](const std::string& v) { return !(v == "0" || v == "false" || v == "False"); };
  for (size_t i = 0; i < args.size(); ++i) {
    std::string a = args[i];
    if (a.empty() || a[0] != '-') { o.rest.push_back(a); continue; }
    size_t p = a.find_first_not_of('-');
    std::string name = a.substr(p), val;
    bool has_val = false;
    size_t eq = name.find('=');
    if (eq != std::string::npos) { val = name.substr(eq + 1); name = name.substr(0, eq); has_val = true; }
    auto next = [&]() -> std::string {
      if (has_val) return val;
      PS_CHECK_LT(i + 1, args.size()) << "flag -" << name << " needs a value";
      return args[++i];
    };
    if (name == "num_servers") o.num_servers = atoi(next().c_str());
    else if (name == "num_workers") o.num_workers = atoi(next().c_str());
    else if (name == "num_threads") o.num_threads = atoi(next().c_str());
    else if (name == "num_replicas") o.num_replicas = atoi(next().c_str());
    else if (name == "my_node") o.my_node = next();
    else if (name == "scheduler") o.scheduler = next();
    else if (name == "interface") o.interface = next();
    else if (name == "app_file") o.app_file = next();
    else if (name == "app_conf") o.app_conf = next();
    else if (name == "key_start") o.key_start = strtoull(next().c_str(), nullptr, 10);
    else if (name == "key_end") o.key_end = strtoull(next().c_str(), nullptr, 10);
    else if (name == "bind_to") o.bind_to = atoi(next().c_str());
    else if (name == "report_interval") o.report_interval = atoi(next().c_str());
    else if (name == "log_dir") o.log_dir = next();
    else if (name == "hash_kernel") o.hash_kernel = strtoull(next().c_str(), nullptr, 10);
    else if (name == "line_limit") o.line_limit = atoi(next().c_str());
    else if (name == "shuffle_fea_id") o.shuffle_fea_id = has_val ? as_bool(val) : true;
    else if (name == "local") o.local = has_val ? as_bool(val) : true;
    else if (name == "logtostderr" || name == "v") { if (!has_val && i + 1 < args.size() && args[i + 1][0] != '-') ++i; }
    else { o.rest.push_back(a); }
  }
  return o;
}

void Options::InitFromEnv() {
  const char* uri = getenv("DMLC_PS_ROOT_URI");
  const char* port = getenv("DMLC_PS_ROOT_PORT");
  if (!uri || !port) return;
  scheduler = std::string("role:SCHEDULER,hostname:'") + uri + "',port:" + port + ",id:'H'";
  if (const char* v = getenv("DMLC_NUM_WORKER")) num_workers = atoi(v);
  if (const char* v = getenv("DMLC_NUM_SERVER")) num_servers = atoi(v);
  std::string role;
  int rank = -1;
  if (const char* v = getenv("DMLC_ROLE")) {
    role = v;
  } else {
    // an MPI launcher: rank 0 is the scheduler, then servers, then workers
    const char* r = getenv("PMI_RANK");
    if (!r) r = getenv("OMPI_COMM_WORLD_RANK");
    if (!r) return;
    rank = atoi(r);
    if (rank == 0) role = "scheduler";
    else if (rank <= num_servers) role = "server";
    else role = "worker";
  }
  if (role == "scheduler") { my_node = scheduler; return; }
  std::string ip = Env::LocalIP(interface);
  int p = Env::FreePort();
  bool server = role == "server";
  std::string id = std::string(server ? "S" : "W") + "_" + ip + "_" + std::to_string(p);
  my_node = std::string("role:") + (server ? "SERVER" : "WORKER") + ",hostname:'" + ip + "',port:" +
            std::to_string(p) + ",id:'" + id + "'";
}

int Env::FreePort() {
  // A port that is free now and stays free until the caller binds it: taken from below the range that the
  // kernel uses for the source ports of outgoing connections (a port from that range, found by binding port 0,
  // can be grabbed by any connect() on the machine before the node that was promised it starts to listen).
  static std::mutex mu;
  static std::set<int> handed_out;
  static std::mt19937 rng((unsigned)std::chrono::steady_clock::now().time_since_epoch().count() ^ (unsigned)getpid());
  int low = 32768;
  if (FILE* f = fopen("/proc/sys/net/ipv4/ip_local_port_range", "r")) {
    int a = 0, b = 0;
    if (fscanf(f, "%d %d", &a, &b) == 2 && a > 0) low = a;
    fclose(f);
  }
  std::lock_guard<std::mutex> l(mu);
  const int first = 10000;
  for (int attempt = 0; low > first + 1000 && attempt < 200; ++attempt) {
    const int port = first + (int)(rng() % (unsigned)(low - first));
    if (handed_out.count(port)) continue;
    int fd = socket(AF_INET, SOCK_STREAM, 0);
    sockaddr_in addr; memset(&addr, 0, sizeof(addr));
    addr.sin_family = AF_INET;
    addr.sin_addr.s_addr = htonl(INADDR_ANY);
    addr.sin_port = htons((uint16_t)port);
    const bool ok = bind(fd, (sockaddr*)&addr, sizeof(addr)) == 0;
    close(fd);
    if (ok) { handed_out.insert(port); return port; }
  }
  // no room below the range: whatever the kernel gives
  int fd = socket(AF_INET, SOCK_STREAM, 0);
  sockaddr_in addr; memset(&addr, 0, sizeof(addr));
  addr.sin_family = AF_INET;
  addr.sin_addr.s_addr = htonl(INADDR_ANY);
  addr.sin_port = 0;
  int port = 0;
  if (bind(fd, (sockaddr*)&addr, sizeof(addr)) == 0) {
    socklen_t len = sizeof(addr);
    if (getsockname(fd, (sockaddr*)&addr, &len) == 0) port = ntohs(addr.sin_port);
  }
  close(fd);
  return port;
}

std::string Env::LocalIP(const std::string& interface) {
  ifaddrs* ifs = nullptr;
  std::string ip = "127.0.0.1";
  if (getifaddrs(&ifs) != 0) return ip;
  for (ifaddrs* i = ifs; i; i = i->ifa_next) {
    if (!i->ifa_addr || i->ifa_addr->sa_family != AF_INET) continue;
    if (!interface.empty() && interface != i->ifa_name) continue;
    if (interface.empty() && (i->ifa_flags & IFF_LOOPBACK)) continue;
    char buf[INET_ADDRSTRLEN];
    inet_ntop(AF_INET, &((sockaddr_in*)i->ifa_addr)->sin_addr, buf, sizeof(buf));
    ip = buf;
    break;
  }
  freeifaddrs(ifs);
  return ip;
}

}  // namespace PS
