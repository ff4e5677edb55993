// The user-facing facade: role queries, system start/stop, and the two entry
// points a "simple" program defines. Counterpart of src/ps.h:15-78 and
// src/ps_main.cc:4-24.
#pragma once
#include "monitor.h"
#include "parameter.h"
#include "postoffice.h"

namespace PS {

// A simple program defines these two: servers are created from
// CreateServerNode, workers run WorkerNodeMain (see ps_main.cc).
int WorkerNodeMain(int argc, char* argv[]);
App* CreateServerNode(const std::string& conf);

inline App* MyApp() { return Postoffice::instance().manager().app(); }
inline Node MyNode() { return Postoffice::instance().manager().van().my_node(); }
inline std::string MyNodeID() { return MyNode().id; }
inline int IsWorker() { return MyNode().role == Node::WORKER; }
inline int IsServer() { return MyNode().role == Node::SERVER; }
inline int IsScheduler() { return MyNode().role == Node::SCHEDULER; }
inline Range<Key> MyKeyRange() { return MyNode().key; }
inline std::string SchedulerID() { return Postoffice::instance().manager().van().scheduler().id; }
inline int NextCustomerID() { return Postoffice::instance().manager().NextCustomerID(); }
// my rank among the nodes of my role, and that group's size
inline int MyRank() { return MyNode().rank; }
inline int RankSize() {
  auto& m = Postoffice::instance().manager();
  return IsWorker() ? m.num_workers() : (IsServer() ? m.num_servers() : 1);
}
inline void WaitServersReady() { Postoffice::instance().manager().WaitServersReady(); }
inline void WaitWorkersReady() { Postoffice::instance().manager().WaitWorkersReady(); }
inline void StartSystem(int argc, char* argv[]) { Postoffice::instance().Run(Options::Parse(argc, argv)); }
inline void StopSystem() { Postoffice::instance().Stop(); }
inline int RunSystem(int argc, char* argv[]) { StartSystem(argc, argv); StopSystem(); return 0; }

}  // namespace PS
