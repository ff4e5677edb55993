// Manager: the control plane of a node -- bootstrap (REQUEST_APP /
// REGISTER_NODE / ADD_NODE), node list, customer registry, readiness counters,
// orderly shutdown (READY_TO_EXIT / EXIT) and node-failure handling
// (REMOVE_NODE). Counterpart of system/manager.h:13-93, system/manager.cc:26-333.
#pragma once
#include <set>
#include "assigner.h"
#include "env.h"
#include "van.h"

namespace PS {

class App;
class Customer;
class Postoffice;

class Manager {
 public:
  explicit Manager(Postoffice* po) : sys_(po) {}
  ~Manager();
  void Init(const Options& opt);
  // blocks until this node is registered (and, for workers, servers are ready); then app->Run()
  void Run(bool run_app = true);
  void Stop();
  void StopCustomers();   // joins the executor threads of all registered customers
  // handles a control message; returns false on EXIT
  bool Process(Message* msg);

  // node list
  void AddNode(const Node& node);
  void RemoveNode(const NodeID& node_id);
  // called by the Van when a peer's connection drops
  void NodeDisconnected(const NodeID& node_id);
  typedef std::function<void(const NodeID&)> NodeFailureHandler;
  void AddNodeFailureHandler(NodeFailureHandler h) { Lock l(nodes_mu_); node_failure_handlers_.push_back(h); }

  // customers
  void AddCustomer(Customer* obj);
  void RemoveCustomer(int id);
  // waits (up to a timeout) for the customer to be registered
  Customer* customer(int id);
  int NextCustomerID();

  void WaitServersReady();
  void WaitWorkersReady();
  int num_workers() { Lock l(nodes_mu_); return num_workers_; }
  int num_servers() { Lock l(nodes_mu_); return num_servers_; }
  // a log of sent requests / received responses would allow resending; these
  // hooks exist for that purpose and only count for now
  void AddRequest(Message* msg) { ++num_requests_; }
  void AddResponse(Message* msg) { ++num_responses_; }

  Van& van() { return van_; }
  App* app() { return app_; }
  bool IsScheduler() const { return van_.my_node().role == Node::SCHEDULER; }
  std::vector<Node> nodes() { Lock l(nodes_mu_); std::vector<Node> v; for (auto& n : nodes_) v.push_back(n.second); return v; }
  bool done() const { return done_; }

 private:
  Task NewControlTask(Control::Command cmd);
  void SendTask(const NodeID& recver, const Task& task);
  void SendTask(const Node& recver, const Task& task) { SendTask(recver.id, task); }
  void CreateApp(const std::string& conf);
  Node my_node() { return van_.my_node(); }

  Postoffice* sys_;
  Options opt_;
  Van van_;
  App* app_ = nullptr;
  std::string app_conf_;
  std::unique_ptr<NodeAssigner> node_assigner_;

  std::mutex nodes_mu_;
  std::condition_variable nodes_cv_;
  std::map<NodeID, Node> nodes_;
  int num_workers_ = 0, num_servers_ = 0;
  int num_active_nodes_ = 0;     // scheduler: nodes that have not said READY_TO_EXIT
  bool is_my_node_inited_ = false;
  std::atomic<bool> done_{false};
  bool in_exit_ = false;
  std::vector<NodeFailureHandler> node_failure_handlers_;
  std::set<NodeID> failure_notified_;   // lost nodes whose handlers have run (guarded by nodes_mu_)

  std::mutex customer_mu_;
  std::condition_variable customer_cv_;
  std::map<int, Customer*> customers_;
  int next_customer_id_ = 1;
  std::atomic<size_t> num_requests_{0}, num_responses_{0};
};

}  // namespace PS
