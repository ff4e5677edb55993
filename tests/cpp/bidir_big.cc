// Large messages in both directions at once: every worker issues pushes (keys + values out) and pulls (keys out,
// values back) of about a million keys each without waiting in between, so that its outgoing streams and the
// servers' replies fill the socket buffers at the same time; everything must still complete. Prints
// "DONE <rounds> <checksum>" on every worker.
#include <cstdio>
#include "ps.h"

namespace PS {

static const int kModel = 3;
static const size_t kKeys = 1000000;
static const int kRounds = 6;

class Server : public App {
 public:
  explicit Server(Postoffice* po) : App(po), model_(false, 1, kModel, po) {}
 private:
  KVVector<Key, float> model_;
};

class Worker : public App {
 public:
  explicit Worker(Postoffice* po) : App(po), model_(false, 1, kModel, po) {}
  void Run() override {
    App::Run();
    SArray<Key> keys(kKeys);
    const Key stride = kMaxKey / kKeys;                 // spread over every server's key range
    for (size_t i = 0; i < kKeys; ++i) keys[i] = i * stride + 7;
    SArray<float> vals(kKeys, 1.f);
    model_[0].key = keys;
    model_[0].value = SArray<float>(kKeys, 0.f);
    std::vector<int> stamps;
    for (int r = 0; r < kRounds; ++r) {
      stamps.push_back(model_.Push(Parameter::Request(0), keys, {vals}));
      stamps.push_back(model_.Pull(Parameter::Request(0), keys));
    }
    for (int ts : stamps) model_.Wait(ts);
    double sum = 0;
    for (size_t i = 0; i < kKeys; i += 1000) sum += model_[0].value[i];
    std::printf("DONE %d %g\n", kRounds, sum);
  }
 private:
  KVVector<Key, float> model_;
};

class Idle : public App {
 public:
  explicit Idle(Postoffice* po) : App(po) {}
};

}  // namespace PS

int main(int argc, char* argv[]) {
  PS::App::SetFactory([](const std::string&, PS::Postoffice* po) -> PS::App* {
    switch (po->manager().van().my_node().role) {
      case PS::Node::SERVER: return new PS::Server(po);
      case PS::Node::WORKER: return new PS::Worker(po);
      default: return new PS::Idle(po);
    }
  });
  return PS::RunSystem(argc, argv);
}
