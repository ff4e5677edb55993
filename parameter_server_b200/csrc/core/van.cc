#include "van.h"

#include <sys/ioctl.h>

#include <arpa/inet.h>
#include <fcntl.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/uio.h>
#include <sys/un.h>
#include <unistd.h>

namespace PS {

std::mutex Van::hub_mu_;
std::map<std::string, std::shared_ptr<Van::InProcEndpoint>> Van::hub_;

static const uint32_t kFrameMagic = 0x50534231;  // "PSB1"
static const int kSocketBufferBytes = 4 << 20;    // asked of the kernel, which caps it at its own limit
static const size_t kDirectSendBytes = 64 << 10;  // what a submitting thread may write itself (see WritableNow)

static bool WriteAll(int fd, const void* p, size_t n) {
  const char* c = (const char*)p;
  while (n) {
    ssize_t w = ::send(fd, c, n, MSG_NOSIGNAL);
    if (w < 0) { if (errno == EINTR) continue; return false; }
    c += w; n -= w;
  }
  return true;
}
static bool ReadAll(int fd, void* p, size_t n) {
  char* c = (char*)p;
  while (n) {
    ssize_t r = ::recv(fd, c, n, 0);
    if (r == 0) return false;
    if (r < 0) { if (errno == EINTR) continue; return false; }
    c += r; n -= r;
  }
  return true;
}

Van::~Van() { Destroy(); }

Node Van::ParseNode(const std::string& s) {
  // comma separated key:value pairs; string values in single quotes
  Node n;
  size_t i = 0;
  while (i < s.size()) {
    size_t c = s.find(':', i);
    if (c == std::string::npos) break;
    std::string key = s.substr(i, c - i);
    while (!key.empty() && (key[0] == ' ' || key[0] == ',')) key.erase(0, 1);
    size_t v0 = c + 1, v1;
    std::string val;
    if (v0 < s.size() && (s[v0] == '\'' || s[v0] == '"')) {
      v1 = s.find(s[v0], v0 + 1);
      PS_CHECK(v1 != std::string::npos) << "unterminated string in node: " << s;
      val = s.substr(v0 + 1, v1 - v0 - 1);
      i = v1 + 1;
    } else {
      v1 = s.find(',', v0);
      if (v1 == std::string::npos) v1 = s.size();
      val = s.substr(v0, v1 - v0);
      i = v1;
    }
    if (i < s.size() && s[i] == ',') ++i;
    if (key == "role") {
      if (val == "SERVER") n.role = Node::SERVER;
      else if (val == "WORKER") n.role = Node::WORKER;
      else if (val == "SCHEDULER") n.role = Node::SCHEDULER;
      else PS_CHECK(false) << "unknown role " << val;
    } else if (key == "hostname") n.hostname = val;
    else if (key == "port") n.port = atoi(val.c_str());
    else if (key == "id") n.id = val;
    else if (key == "rank") n.rank = atoi(val.c_str());
  }
  if (n.id.empty()) {
    // synthesise an id from the address, prefixed by the role letter
    const char* pre = n.role == Node::SERVER ? "S" : n.role == Node::WORKER ? "W" : "H";
    n.id = std::string(pre) + "_" + n.hostname + "_" + std::to_string(n.port);
  }
  return n;
}

void Van::Init(const Node& my_node, const Node& scheduler, bool local_ipc) {
  my_node_ = my_node;
  scheduler_ = scheduler;
  local_ipc_ = local_ipc;
  inproc_ = my_node.hostname == "inproc";
  running_ = true;
  if (inproc_) {
    my_endpoint_ = std::make_shared<InProcEndpoint>();
    Lock l(hub_mu_);
    hub_[address(my_node_)] = my_endpoint_;
  } else {
    PS_CHECK_EQ(pipe(wake_fd_), 0);
    if (local_ipc_) {
      listen_fd_ = socket(AF_UNIX, SOCK_STREAM, 0);
      sockaddr_un addr; memset(&addr, 0, sizeof(addr));
      addr.sun_family = AF_UNIX;
      std::string path = "/tmp/psb_" + std::to_string(my_node_.port);
      unlink(path.c_str());
      strncpy(addr.sun_path, path.c_str(), sizeof(addr.sun_path) - 1);
      PS_CHECK_EQ(bind(listen_fd_, (sockaddr*)&addr, sizeof(addr)), 0) << "bind " << path;
    } else {
      listen_fd_ = socket(AF_INET, SOCK_STREAM, 0);
      int one = 1;
      setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
      // accepted streams inherit this: room for a few whole messages, so that a sender's write returns
      // while the poll thread is still busy with another peer
      int rcv = kSocketBufferBytes;
      setsockopt(listen_fd_, SOL_SOCKET, SO_RCVBUF, &rcv, sizeof(rcv));
      sockaddr_in addr; memset(&addr, 0, sizeof(addr));
      addr.sin_family = AF_INET;
      addr.sin_addr.s_addr = htonl(INADDR_ANY);
      addr.sin_port = htons((uint16_t)my_node_.port);
      PS_CHECK_EQ(bind(listen_fd_, (sockaddr*)&addr, sizeof(addr)), 0)
          << "bind to port " << my_node_.port << " failed: " << strerror(errno);
    }
    PS_CHECK_EQ(listen(listen_fd_, 256), 0);
    poll_thread_ = std::thread([this] { PollLoop(); });
  }
  Connect(scheduler_);
  if (my_node_.id != scheduler_.id) Connect(my_node_);
}

void Van::Destroy() {
  if (!running_) return;
  running_ = false;
  if (inproc_) {
    Lock l(hub_mu_);
    hub_.erase(address(my_node_));
  } else {
    char c = 'x';
    if (wake_fd_[1] >= 0) { ssize_t r = write(wake_fd_[1], &c, 1); (void)r; }
    if (poll_thread_.joinable()) poll_thread_.join();
    Lock l(mu_);
    for (auto& it : senders_) close(it.second);
    senders_.clear();
    if (listen_fd_ >= 0) close(listen_fd_);
    close(wake_fd_[0]); close(wake_fd_[1]);
    if (local_ipc_) unlink(("/tmp/psb_" + std::to_string(my_node_.port)).c_str());
  }
}

bool Van::Connect(const Node& node) {
  PS_CHECK(!node.id.empty());
  Lock l(mu_);
  { Lock n(names_mu_); hostnames_[node.id] = node.hostname; }
  if (inproc_) {
    if (in_senders_.count(node.id)) return true;
    // the peer may not have bound yet: wait briefly
    for (int i = 0; i < 2000; ++i) {
      {
        Lock h(hub_mu_);
        auto it = hub_.find(address(node));
        if (it != hub_.end()) { in_senders_[node.id] = it->second; return true; }
      }
      std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
    PS_LOG(WARN) << my_node_.id << ": inproc peer " << node.id << " not found";
    return false;
  }
  if (senders_.count(node.id)) return true;
  int fd = -1;
  for (int attempt = 0; attempt < 600; ++attempt) {   // the peer may still be starting
    if (local_ipc_) {
      fd = socket(AF_UNIX, SOCK_STREAM, 0);
      sockaddr_un addr; memset(&addr, 0, sizeof(addr));
      addr.sun_family = AF_UNIX;
      std::string path = "/tmp/psb_" + std::to_string(node.port);
      strncpy(addr.sun_path, path.c_str(), sizeof(addr.sun_path) - 1);
      if (connect(fd, (sockaddr*)&addr, sizeof(addr)) == 0) break;
    } else {
      fd = socket(AF_INET, SOCK_STREAM, 0);
      int snd = kSocketBufferBytes;
      setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &snd, sizeof(snd));
      sockaddr_in addr; memset(&addr, 0, sizeof(addr));
      addr.sin_family = AF_INET;
      addr.sin_port = htons((uint16_t)node.port);
      if (inet_pton(AF_INET, node.hostname.c_str(), &addr.sin_addr) != 1) {
        hostent* he = gethostbyname(node.hostname.c_str());
        PS_CHECK(he != nullptr) << "cannot resolve " << node.hostname;
        memcpy(&addr.sin_addr, he->h_addr_list[0], he->h_length);
      }
      if (connect(fd, (sockaddr*)&addr, sizeof(addr)) == 0) {
        int one = 1;
        setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
        break;
      }
    }
    close(fd); fd = -1;
    std::this_thread::sleep_for(std::chrono::milliseconds(50));
  }
  if (fd < 0) { PS_LOG(WARN) << my_node_.id << ": cannot connect to " << node.ShortDebugString(); return false; }
  // identify myself (the counterpart of a socket identity)
  uint32_t hello[2] = {kFrameMagic, (uint32_t)my_node_.id.size()};
  if (!WriteAll(fd, hello, sizeof(hello)) || !WriteAll(fd, my_node_.id.data(), my_node_.id.size())) {
    close(fd); return false;
  }
  senders_[node.id] = fd;
  PS_VLOG(1) << my_node_.id << " connected to " << node.id;
  return true;
}

bool Van::Disconnect(const Node& node) {
  Lock l(mu_);
  in_senders_.erase(node.id);
  auto it = senders_.find(node.id);
  if (it != senders_.end()) { close(it->second); senders_.erase(it); }
  return true;
}

bool Van::Send(Message* msg, size_t* send_bytes) {
  const NodeID& id = msg->recver;
  size_t data_size = msg->key.size();
  for (auto& v : msg->value) data_size += v.size();
  msg->task.has_key = !msg->key.empty();
  bool ok = false;
  if (inproc_) {
    std::shared_ptr<InProcEndpoint> ep;
    {
      Lock l(mu_);
      auto it = in_senders_.find(id);
      if (it != in_senders_.end()) ep = it->second;
    }
    if (!ep) { PS_LOG(WARN) << my_node_.id << ": no channel to " << id; return false; }
    auto copy = std::make_shared<Message>(*msg);  // shares the payload buffers
    copy->sender = my_node_.id;
    copy->callback = nullptr;
    ep->queue.push(copy);
    data_size += 64;
    ok = true;
  } else {
    std::string header = msg->task.Serialize();
    Lock l(mu_);
    auto it = senders_.find(id);
    if (it == senders_.end()) { PS_LOG(WARN) << my_node_.id << ": no channel to " << id; return false; }
    ok = SendTcp(it->second, header, msg);
    data_size += header.size();
  }
  *send_bytes = data_size;
  if (IsLocalPeer(id)) sent_to_local_ += data_size;
  else sent_to_others_ += data_size;
  PS_VLOG(2) << "send " << msg->ShortDebugString();
  return ok;
}

bool Van::WritableNow(const NodeID& id, size_t bytes) {
  if (inproc_) return true;
  if (bytes > kDirectSendBytes) return false;
  std::unique_lock<std::mutex> l(mu_, std::try_to_lock);
  if (!l.owns_lock()) return false;           // somebody is writing: do not wait for it
  auto it = senders_.find(id);
  if (it == senders_.end()) return false;
  int unsent = 0;
  return ioctl(it->second, TIOCOUTQ, &unsent) == 0 && unsent == 0;
}

bool Van::SendTcp(int fd, const std::string& header, Message* msg) {
  // [magic][nframes][len...] then the frames: header, (key), values...
  std::vector<uint64_t> lens;
  std::vector<iovec> iov;
  lens.push_back(header.size());
  if (msg->task.has_key) lens.push_back(msg->key.size());
  for (auto& v : msg->value) lens.push_back(v.size());
  uint32_t head[2] = {kFrameMagic, (uint32_t)lens.size()};
  iov.push_back({head, sizeof(head)});
  iov.push_back({lens.data(), lens.size() * sizeof(uint64_t)});
  iov.push_back({(void*)header.data(), header.size()});
  if (msg->task.has_key) iov.push_back({msg->key.data(), msg->key.size()});
  for (auto& v : msg->value) if (v.size()) iov.push_back({v.data(), v.size()});
  size_t idx = 0;
  while (idx < iov.size()) {
    msghdr mh; memset(&mh, 0, sizeof(mh));
    mh.msg_iov = &iov[idx];
    mh.msg_iovlen = std::min<size_t>(iov.size() - idx, 64);
    ssize_t w = sendmsg(fd, &mh, MSG_NOSIGNAL);
    if (w < 0) { if (errno == EINTR) continue; return false; }
    size_t left = (size_t)w;
    while (idx < iov.size() && left >= iov[idx].iov_len) { left -= iov[idx].iov_len; ++idx; }
    if (idx < iov.size() && left) { iov[idx].iov_base = (char*)iov[idx].iov_base + left; iov[idx].iov_len -= left; }
  }
  return true;
}

bool Van::RecvTcp(int fd, Message* msg, size_t* bytes) {
  uint32_t head[2];
  if (!ReadAll(fd, head, sizeof(head))) return false;
  if (head[0] != kFrameMagic || head[1] == 0 || head[1] > 4096) return false;
  std::vector<uint64_t> lens(head[1]);
  if (!ReadAll(fd, lens.data(), lens.size() * sizeof(uint64_t))) return false;
  std::string header(lens[0], '\0');
  if (!ReadAll(fd, &header[0], lens[0])) return false;
  if (!msg->task.Parse(header.data(), header.size())) return false;
  *bytes = header.size();
  size_t f = 1;
  msg->key.clear(); msg->value.clear();
  if (msg->task.has_key) {
    PS_CHECK_LT(f, lens.size());
    SArray<char> k(lens[f]);
    if (lens[f] && !ReadAll(fd, k.data(), lens[f])) return false;
    msg->key = k; *bytes += lens[f]; ++f;
  }
  for (; f < lens.size(); ++f) {
    SArray<char> v(lens[f]);
    if (lens[f] && !ReadAll(fd, v.data(), lens[f])) return false;
    msg->value.push_back(v); *bytes += lens[f];
  }
  return true;
}

void Van::PollLoop() {
  std::vector<int> fds;  // accepted peer streams
  while (running_) {
    std::vector<pollfd> p;
    p.push_back({listen_fd_, POLLIN, 0});
    p.push_back({wake_fd_[0], POLLIN, 0});
    for (int fd : fds) p.push_back({fd, POLLIN, 0});
    int r = poll(p.data(), p.size(), 500);
    if (r < 0) { if (errno == EINTR) continue; break; }
    if (!running_) break;
    if (p[1].revents & POLLIN) { char c; ssize_t n = read(wake_fd_[0], &c, 1); (void)n; }
    if (p[0].revents & POLLIN) {
      int fd = accept(listen_fd_, nullptr, nullptr);
      if (fd >= 0) {
        uint32_t hello[2];
        std::string id;
        if (ReadAll(fd, hello, sizeof(hello)) && hello[0] == kFrameMagic && hello[1] < 256) {
          id.resize(hello[1]);
          if (ReadAll(fd, &id[0], hello[1])) { fds.push_back(fd); fd_to_id_[fd] = id; }
          else close(fd);
        } else close(fd);
      }
    }
    for (size_t i = 2; i < p.size(); ++i) {
      if (!(p[i].revents & (POLLIN | POLLHUP | POLLERR))) continue;
      int fd = p[i].fd;
      auto m = std::make_shared<Message>();
      size_t bytes = 0;
      NodeID id;
      // (no lock: only this thread uses the map, and the lock of the senders must not be waited for here:
      // a send thread blocked in a write holds it until the peer reads, and the peer reads only while its
      // own poll thread runs)
      id = fd_to_id_[fd];
      if (RecvTcp(fd, m.get(), &bytes)) {
        m->sender = id;
        m->recver = my_node_.id;
        if (IsLocalPeer(id)) received_from_local_ += bytes;
        else received_from_others_ += bytes;
        Deliver(m);
      } else {
        // EOF or a broken stream: the peer is gone
        close(fd);
        fds.erase(std::find(fds.begin(), fds.end(), fd));
        fd_to_id_.erase(fd);
        if (running_ && on_disconnect_ && !id.empty()) on_disconnect_(id);
      }
    }
  }
  for (int fd : fds) close(fd);
}

void Van::Deliver(const MessagePtr& m) {
  ULock l(deliver_mu_);
  if (sink_ && direct_ok_ && inbox_.empty() && !recv_busy_) {
    PS_VLOG(2) << "recv " << m->ShortDebugString();
    sink_(m);        // under the lock: Recv() cannot take a later message meanwhile
    return;
  }
  inbox_.push_back(m);
  deliver_cv_.notify_one();
}

bool Van::Recv(Message* msg, size_t* recv_bytes) {
  MessagePtr m;
  if (inproc_) {
    my_endpoint_->queue.wait_and_pop(m);
  } else {
    ULock l(deliver_mu_);
    recv_busy_ = false;              // the caller is done with the message before
    deliver_cv_.wait(l, [this] { return !inbox_.empty(); });
    m = inbox_.front();
    inbox_.pop_front();
    recv_busy_ = !m->terminate;
  }
  *msg = *m;
  msg->recver = my_node_.id;
  size_t n = msg->key.size() + 64;
  for (auto& v : msg->value) n += v.size();
  *recv_bytes = n;
  if (inproc_) received_from_local_ += n;
  PS_VLOG(2) << "recv " << msg->ShortDebugString();
  return !msg->terminate;
}

void Van::WakeUp() {
  auto m = std::make_shared<Message>();
  m->terminate = true;
  m->sender = my_node_.id;
  if (inproc_) { my_endpoint_->queue.push(m); return; }
  Lock l(deliver_mu_);
  inbox_.push_back(m);
  deliver_cv_.notify_one();
}

std::string Van::Statistic() const {
  auto gb = [](size_t x) { return x / 1e9; };
  std::ostringstream ss;
  ss << my_node_.id << " sent " << gb(sent_to_local_ + sent_to_others_) << " (local " << gb(sent_to_local_)
     << ") GB, received " << gb(received_from_local_ + received_from_others_) << " (local "
     << gb(received_from_local_) << ") GB";
  return ss.str();
}

}  // namespace PS
