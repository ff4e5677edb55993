// Raw message throughput of the host transport over real sockets: every worker sends `-n` requests
// that carry `-data_size` KB of payload to every server and waits for each to be acknowledged; it
// prints MB/s of payload (what the reference's src/test/network_perf_ps.cc:23-47 reports). A program
// with its own main(): it registers an application factory and runs the system.
//
//   make examples
//   python -m parameter_server_b200.system.launch start -ns 2 -nw 2 -- build/network_perf -n=200 -data_size=1000
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include "evaluation.h"
#include "ps.h"

namespace {
int flag(int argc, char** argv, const char* name, int dflt) {
  size_t len = strlen(name);
  for (int i = 1; i < argc; ++i) {
    const char* a = argv[i];
    while (*a == '-') ++a;
    if (strncmp(a, name, len) == 0 && a[len] == '=') return atoi(a + len + 1);
  }
  return dflt;
}
}  // namespace

namespace PS {

class Sender : public App {
 public:
  Sender(Postoffice* po, int n, int kb) : App(po), n_(n), kb_(kb) {}
  // every server gets the whole payload, not a key-range slice of it
  void Slice(const Message& request, const std::vector<Range<Key>>&, std::vector<Message*>* msgs) override {
    for (auto* m : *msgs) *m = request;
  }
  void Run() override {
    App::Run();
    SArray<int> payload(size_t(kb_) * 1000 / sizeof(int), 1);
    auto start = tic();
    for (int i = 0; i < n_; ++i) {
      Message msg;
      msg.add_value(payload);
      msg.recver = kServerGroup;
      Wait(Submit(&msg));
    }
    double sec = toc(start);
    int servers = Postoffice::instance().manager().num_servers();
    std::printf("%s: packet size %d KB to %d servers, %d rounds, throughput %.1f MB/s\n", MyNodeID().c_str(), kb_,
                servers, n_, double(kb_) / 1000.0 * n_ * servers / sec);
  }
 private:
  int n_, kb_;
};

class Idle : public App {
 public:
  explicit Idle(Postoffice* po) : App(po) {}
};

}  // namespace PS

int main(int argc, char* argv[]) {
  int n = flag(argc, argv, "n", 200), kb = flag(argc, argv, "data_size", 1000);
  PS::App::SetFactory([n, kb](const std::string&, PS::Postoffice* po) -> PS::App* {
    if (po->manager().van().my_node().role == PS::Node::WORKER) return new PS::Sender(po, n, kb);
    return new PS::Idle(po);
  });
  return PS::RunSystem(argc, argv);
}
