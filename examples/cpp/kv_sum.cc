// A "simple" parameter-server program in C++: it defines only the two entry points that
// ps_main.cc asks for. Every server keeps a map whose entries add what is pushed; every worker
// pushes its values under three keys, pulls the sums after its own push and prints them.
// (The shape of the reference's src/test/kv_map_ps.cc and hello_ps.cc, written against this
// framework's headers.)
//
//   make examples && python -m parameter_server_b200.system.launch start -ns 2 -nw 2 -- build/kv_sum
#include <unistd.h>
#include <cstdio>
#include "ps.h"

namespace PS {

struct AddEntry {
  float v = 0;
  void Get(float* data, void*) const { *data = v; }
  void Set(const float* data, void*) { v += *data; }
};
struct Nothing { void Update() {} };

static const int kModelId = 7;   // the same customer id on every node names the same shared object

class SumServer : public App {
 public:
  SumServer() : model_(1, kModelId) {}
 private:
  KVMap<Key, float, AddEntry, Nothing> model_;
};

App* CreateServerNode(const std::string& conf) { return new SumServer(); }

int WorkerNodeMain(int argc, char* argv[]) {
  KVVector<Key, float> model(false, 1, kModelId);
  const Key half = Key(1) << 63;                    // with two servers the third key lives on the second
  SArray<Key> keys{3, 11, half + 4};
  float scale = float(MyRank() + 1);
  SArray<float> vals{1 * scale, 2 * scale, 3 * scale};
  model[0].key = keys;
  model[0].value = SArray<float>(keys.size(), 0.f);

  int pushed = model.Push(Parameter::Request(0), keys, {vals});
  model.Wait(pushed);
  // the pull names this worker's push in its wait list, so the servers answer it after that push; the other
  // workers push whenever they get there (nothing synchronises workers here), so pull until their share is in
  int n = RankSize();
  float want = 0;
  for (int r = 1; r <= n; ++r) want += float(r);
  for (int attempt = 0; attempt < 200; ++attempt) {
    int pulled = model.Pull(Parameter::Request(0, Message::kInvalidTime, {pushed}), keys);
    model.Wait(pulled);
    if (model[0].value[0] == want) break;
    usleep(10000);
  }
  std::printf("%s pulled %g %g %g\n", MyNodeID().c_str(), model[0].value[0], model[0].value[1], model[0].value[2]);
  return model[0].value[2] == 3 * want ? 0 : 1;
}

}  // namespace PS
