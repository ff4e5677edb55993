// Executor: the per-customer DAG engine. It stamps and slices outgoing
// requests, keeps per-peer timestamp trackers, and runs one thread that picks
// the next *runnable* received message: a response, or a request whose every
// wait_time of the same sender is finished. This is what gives BSP, bounded
// delay and full asynchrony out of one mechanism.
// Counterpart of system/executor.h:22-104, system/executor.cc:16-375.
#pragma once
#include <list>
#include "remote_node.h"

namespace PS {

// virtual group ids (system/executor.h:6-18)
static const NodeID kServerGroup = "all_servers";
static const NodeID kWorkerGroup = "all_workers";
static const NodeID kCompGroup = "all_comp_nodes";    // servers + workers
static const NodeID kReplicaGroup = "all_replicas";   // nodes replicating my key range
static const NodeID kOwnerGroup = "all_owners";       // nodes whose key range I replicate
static const NodeID kLiveGroup = "all_lives";         // everyone, scheduler included

class Customer;
class Postoffice;

class Executor {
 public:
  Executor(Customer& obj, Postoffice* sys);
  ~Executor();
  void Start();  // registers with the node and starts the thread
  void Stop();

  int Submit(Message* msg);
  void Reply(Message* request, Message* response);
  // called by the node's receive thread
  void Accept(Message* msg);

  void WaitSentReq(int timestamp);
  void WaitRecvReq(int timestamp, const NodeID& sender);
  void FinishRecvReq(int timestamp, const NodeID& sender);
  int QueryRecvReq(int timestamp, const NodeID& sender);

  std::shared_ptr<Message> last_request() { Lock l(node_mu_); return last_request_; }
  std::shared_ptr<Message> last_response() { Lock l(node_mu_); return last_response_; }
  int time() { Lock l(node_mu_); return time_; }

  void AddNode(const Node& node);
  void RemoveNode(const Node& node);
  void ReplaceNode(const Node& old_node, const Node& new_node);
  // number of live members of a group (or 0/1 for a node)
  int NumAlive(const NodeID& id);

 private:
  void Run();
  bool PickActiveMsg();
  void ProcessActiveMsg();
  bool CheckFinished(RemoteNode* rnode, int timestamp, bool sent);
  int NumFinished(RemoteNode* rnode, int timestamp, bool sent);
  RemoteNode* GetRNode(const NodeID& id);

  Customer& obj_;
  Postoffice* sys_;
  Node my_node_;
  int num_replicas_ = 0;

  std::list<std::shared_ptr<Message>> recv_msgs_;
  std::mutex msg_mu_;
  std::shared_ptr<Message> active_msg_, last_request_, last_response_;
  std::condition_variable dag_cond_;

  std::unordered_map<NodeID, RemoteNode> nodes_;
  std::mutex node_mu_;
  std::condition_variable sent_req_cond_, recv_req_cond_;

  struct ReqInfo {
    NodeID recver;
    std::function<void()> callback;
  };
  std::unordered_map<int, ReqInfo> sent_reqs_;
  int time_ = Message::kInvalidTime;
  bool done_ = false, started_ = false;
  std::thread thread_;
};

}  // namespace PS
