// The user-facing facade: role queries, system start/stop, and the two entry
// points a "simple" program defines. Counterpart of src/ps.h:15-78 and
// src/ps_main.cc:4-24: the free functions keep the reference's names so that
// programs written against it compile unchanged; all of them go through the
// process-wide node (Postoffice::instance()).
#pragma once
#include "monitor.h"
#include "parameter.h"
#include "postoffice.h"

namespace PS {

// A simple program defines these two: servers are created from
// CreateServerNode, workers run WorkerNodeMain (see ps_main.cc).
int WorkerNodeMain(int argc, char* argv[]);
App* CreateServerNode(const std::string& conf);

namespace facade {
inline Manager& manager() { return Postoffice::instance().manager(); }
inline const Node& me() { return manager().van().my_node(); }
inline bool has_role(Node::Role r) { return me().role == r; }
}  // namespace facade

// ---- life cycle
inline void StartSystem(int argc, char* argv[]) { Postoffice::instance().Run(Options::Parse(argc, argv)); }
inline void StopSystem() { Postoffice::instance().Stop(); }
inline int RunSystem(int argc, char* argv[]) {
  StartSystem(argc, argv);
  StopSystem();
  return 0;
}
inline void WaitServersReady() { facade::manager().WaitServersReady(); }
inline void WaitWorkersReady() { facade::manager().WaitWorkersReady(); }

// ---- who am I
inline Node MyNode() { return facade::me(); }
inline std::string MyNodeID() { return facade::me().id; }
inline Range<Key> MyKeyRange() { return facade::me().key; }
inline int IsScheduler() { return facade::has_role(Node::SCHEDULER); }
inline int IsServer() { return facade::has_role(Node::SERVER); }
inline int IsWorker() { return facade::has_role(Node::WORKER); }
// rank among the nodes of my role, and how many of them there are
inline int MyRank() { return facade::me().rank; }
inline int RankSize() {
  if (IsWorker()) return facade::manager().num_workers();
  if (IsServer()) return facade::manager().num_servers();
  return 1;
}

// ---- the rest of the job
inline App* MyApp() { return facade::manager().app(); }
inline std::string SchedulerID() { return facade::manager().van().scheduler().id; }
inline int NextCustomerID() { return facade::manager().NextCustomerID(); }

}  // namespace PS
