// Server-side aggregation with a virtual timestamp, the bulk-synchronous idiom of the framework: workers push
// two values per key into a buffered vector; the server waits until the push with that timestamp has arrived
// from every worker, folds the buffer into its model and then declares the next timestamp finished; the workers'
// pulls name that timestamp in their wait list, so they are answered only after the aggregation. (The flow of
// the reference's src/test/kv_vector_buffer_ps.cc and aggregation_ps.cc, written against this tree's headers.)
//
//   make examples && python -m parameter_server_b200.system.launch start -ns 1 -nw 2 -- build/aggregation
#include <cstdio>
#include "ps.h"

namespace PS {

static const int kModel = 5;       // customer id of the shared vector on every node
static const int kChannel = 2;     // key channel of the requests
static const int kWidth = 2;       // values per key

class Aggregator : public App {
 public:
  explicit Aggregator(Postoffice* po) : App(po), model_(/*buffer_value=*/true, kWidth, kModel, po) {
    model_[kChannel].key = SArray<Key>{1, 2, 4, 5, 6};      // the union of what the workers will send
  }
  void Run() override {
    App::Run();
    const int push_time = 0;                                // the first request of every worker
    model_.WaitReceivedRequest(push_time, kWorkerGroup);    // every worker's push is in buffer(push_time), summed
    auto& got = model_.buffer(push_time);
    SArray<float> sum(got.values[0].size(), 0.f);
    for (auto& part : got.values) for (size_t i = 0; i < sum.size(); ++i) sum[i] += part[i];
    model_[kChannel].value = sum;
    model_.FinishReceivedRequest(push_time + 1, kWorkerGroup);   // nobody sent this one: it only releases the pulls
  }
 private:
  KVVector<Key, float> model_;
};

class Pusher : public App {
 public:
  explicit Pusher(Postoffice* po) : App(po), model_(false, kWidth, kModel, po) {}
  void Run() override {
    App::Run();
    // different key sets per worker; per key the two pushed arrays hold (1, 2) and (3, 4)
    SArray<Key> keys = MyRank() == 0 ? SArray<Key>{1, 4, 5, 6} : SArray<Key>{1, 2, 4, 5};
    SArray<float> a(keys.size() * kWidth), b(keys.size() * kWidth);
    for (size_t i = 0; i < keys.size(); ++i) { a[2 * i] = 1; a[2 * i + 1] = 2; b[2 * i] = 3; b[2 * i + 1] = 4; }
    int ts = model_.Push(Parameter::Request(kChannel), keys, {a, b});
    model_[kChannel].key = keys;
    model_[kChannel].value = SArray<float>(keys.size() * kWidth, 0.f);
    model_.Wait(model_.Pull(Parameter::Request(kChannel, ts + 2, {ts + 1}), keys));
    std::printf("%s pulled", MyNodeID().c_str());
    for (size_t i = 0; i < model_[kChannel].value.size(); ++i) std::printf(" %g", model_[kChannel].value[i]);
    std::printf("\n");
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
      case PS::Node::SERVER: return new PS::Aggregator(po);
      case PS::Node::WORKER: return new PS::Pusher(po);
      default: return new PS::Idle(po);
    }
  });
  return PS::RunSystem(argc, argv);
}
