// Two threads of a worker submit bursts of small requests to the server without waiting in between; the server
// checks that the requests of the worker arrive with increasing timestamps (a message may be written by the
// submitting thread or by the send thread, and the two paths must not overtake one another), and the worker
// checks that every request was acknowledged. Prints "ORDER OK <n>" on the server and "ACKED <n>" on the worker.
#include <atomic>
#include <cstdio>
#include <thread>
#include "ps.h"

namespace PS {

static const int kPerThread = 3000;

class Checker : public App {
 public:
  explicit Checker(Postoffice* po) : App(po) {}
  void ProcessRequest(Message* msg) override {
    const int t = msg->task.time;
    if (t <= last_) bad_++;
    last_ = t;
    if (++seen_ == 2 * kPerThread) std::printf("%s %d\n", bad_ == 0 ? "ORDER OK" : "ORDER BROKEN", seen_);
  }
 private:
  int last_ = -1, seen_ = 0, bad_ = 0;
};

class Burst : public App {
 public:
  explicit Burst(Postoffice* po) : App(po) {}
  void Run() override {
    App::Run();
    std::atomic<int> last_ts{0};
    auto burst = [&] {
      for (int i = 0; i < kPerThread; ++i) {
        Message msg;
        msg.task.msg = "x";
        msg.recver = kServerGroup;
        int ts = Submit(&msg);
        int seen = last_ts.load();
        while (ts > seen && !last_ts.compare_exchange_weak(seen, ts)) {}
      }
    };
    std::thread a(burst), b(burst);
    a.join(); b.join();
    for (int ts = 0; ts <= last_ts.load(); ++ts) Wait(ts);
    std::printf("ACKED %d\n", last_ts.load() + 1);
  }
};

class Idle : public App {
 public:
  explicit Idle(Postoffice* po) : App(po) {}
};

}  // namespace PS

int main(int argc, char* argv[]) {
  PS::App::SetFactory([](const std::string&, PS::Postoffice* po) -> PS::App* {
    switch (po->manager().van().my_node().role) {
      case PS::Node::SERVER: return new PS::Checker(po);
      case PS::Node::WORKER: return new PS::Burst(po);
      default: return new PS::Idle(po);
    }
  });
  return PS::RunSystem(argc, argv);
}
