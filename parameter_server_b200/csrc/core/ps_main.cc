// Alternative main for "simple" programs that only define
// PS::CreateServerNode and PS::WorkerNodeMain (the reference's src/ps_main.cc:4-24):
// servers run the app returned by CreateServerNode, workers run WorkerNodeMain,
// the scheduler just coordinates start-up and shutdown.
#include "ps.h"

namespace PS {
namespace {
class SimpleWorkerApp : public App {
 public:
  SimpleWorkerApp(Postoffice* po, int argc, char** argv) : App(po), argc_(argc), argv_(argv) {}
  void Run() override { App::Run(); WorkerNodeMain(argc_, argv_); }
 private:
  int argc_;
  char** argv_;
};
class IdleApp : public App {
 public:
  explicit IdleApp(Postoffice* po) : App(po) {}
};
}  // namespace

int SimpleMain(int argc, char* argv[]) {
  App::SetFactory([argc, argv](const std::string& conf, Postoffice* po) -> App* {
    Node::Role role = po->manager().van().my_node().role;
    if (role == Node::SERVER) { App* a = CreateServerNode(conf); return a ? a : new IdleApp(po); }
    if (role == Node::WORKER) return new SimpleWorkerApp(po, argc, argv);
    return new IdleApp(po);
  });
  return RunSystem(argc, argv);
}
}  // namespace PS

#ifdef PSB_SIMPLE_MAIN
int main(int argc, char* argv[]) { return PS::SimpleMain(argc, argv); }
#endif
