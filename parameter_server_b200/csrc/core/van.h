// Van: the host control-plane transport. It moves Messages (Task header + key +
// value byte arrays) between nodes. Counterpart of system/van.h:12-72 and
// system/van.cc:27-330, redesigned without ZeroMQ:
//
//   * "tcp"    -- one listening socket per node, one outgoing stream socket per
//                 peer, length-prefixed frames written with a single writev;
//                 a poll() loop on the receiving side doubles as the
//                 disconnect monitor (EOF on a peer's stream => NodeDisconnected);
//   * "inproc" -- nodes living in the same process (hostname "inproc") hand
//                 messages over through an in-memory hub, sharing the payload
//                 buffers (true zero copy). Used by unit tests and by the
//                 single-process GPU deployment, where the bulk data moves over
//                 NVLink and only headers pass through the Van.
#pragma once
#include <atomic>
#include <set>
#include "message.h"
#include "threading.h"

namespace PS {

class Van {
 public:
  typedef std::function<void(const NodeID&)> DisconnectHandler;
  Van() {}
  ~Van();
  PS_DISALLOW_COPY(Van);

  // bind my endpoint and connect to the scheduler
  void Init(const Node& my_node, const Node& scheduler, bool local_ipc = false);
  void Destroy();
  // open an outgoing channel to `node` (idempotent)
  bool Connect(const Node& node);
  bool Disconnect(const Node& node);
  // returns false on failure; *send_bytes gets the payload size
  bool Send(Message* msg, size_t* send_bytes);
  // blocks until a message arrives; false when the van is shutting down
  bool Recv(Message* msg, size_t* recv_bytes);
  // unblocks Recv (delivers a terminate message to myself)
  void WakeUp();

  const Node& my_node() const { return my_node_; }
  // the scheduler assigns rank and key range after registration
  void UpdateMyNode(const Node& n) { my_node_.rank = n.rank; my_node_.key = n.key; }
  const Node& scheduler() const { return scheduler_; }
  void set_disconnect_handler(DisconnectHandler h) { on_disconnect_ = std::move(h); }
  // tcp: with a sink, and once enable_sink() has been called, the poll thread hands a complete message to the
  // sink as it arrives instead of queueing it for Recv(): one thread hand-over less per message. It does so
  // only while nothing is queued and the thread that calls Recv() is back in Recv(), so messages are handled
  // in their order of arrival and never two at a time. The sink runs on the poll thread and must not block on
  // a peer (it may queue messages, not write them to sockets). Set before Init().
  // true if `bytes` more can be written to the channel to `id` at once without waiting for the peer (nothing
  // of what was written before is still unsent and the message is far smaller than the socket buffer)
  bool WritableNow(const NodeID& id, size_t bytes);
  typedef std::function<void(const MessagePtr&)> Sink;
  void set_sink(Sink s) { sink_ = std::move(s); }
  void enable_sink() { direct_ok_ = true; }
  // "sent x MB (y local), received ..." summary, as printed at exit
  std::string Statistic() const;
  size_t sent_bytes() const { return sent_to_local_ + sent_to_others_; }
  size_t received_bytes() const { return received_from_local_ + received_from_others_; }

  // parses "role:SERVER,hostname:'127.0.0.1',port:8001,id:'S0'"
  static Node ParseNode(const std::string& node_str);
  static std::string address(const Node& n) { return n.hostname + ":" + std::to_string(n.port); }

 private:
  struct InProcEndpoint {
    ThreadsafeQueue<MessagePtr> queue;
  };
  static std::mutex hub_mu_;
  static std::map<std::string, std::shared_ptr<InProcEndpoint>> hub_;

  bool SendTcp(int fd, const std::string& header, Message* msg);
  bool RecvTcp(int fd, Message* msg, size_t* bytes);
  void PollLoop();
  bool IsLocal(const Node& n) const { return n.hostname == my_node_.hostname; }
  // whether peer `id` runs on this host. hostnames_ has a lock of its own that is never held across a write:
  // the poll thread asks this for every message and must not wait for a sender that is blocked on the peer
  bool IsLocalPeer(const NodeID& id) {
    std::lock_guard<std::mutex> l(names_mu_);
    auto h = hostnames_.find(id);
    return h != hostnames_.end() && h->second == my_node_.hostname;
  }

  Node my_node_, scheduler_;
  bool inproc_ = false, local_ipc_ = false;
  std::atomic<bool> running_{false};   // read by the poll thread, written by Destroy()
  int listen_fd_ = -1;
  int wake_fd_[2] = {-1, -1};
  std::mutex mu_;
  std::map<NodeID, int> senders_;                                 // tcp: peer id -> fd
  std::map<NodeID, std::shared_ptr<InProcEndpoint>> in_senders_;  // inproc peers
  std::mutex names_mu_;
  std::map<NodeID, std::string> hostnames_;
  std::shared_ptr<InProcEndpoint> my_endpoint_;
  std::thread poll_thread_;
  // tcp: complete messages from PollLoop that wait for Recv()
  std::mutex deliver_mu_;
  std::condition_variable deliver_cv_;
  std::deque<MessagePtr> inbox_;
  bool recv_busy_ = false;                // the Recv() caller is handling the message it took last
  std::atomic<bool> direct_ok_{false};
  void Deliver(const MessagePtr& m);
  std::map<int, NodeID> fd_to_id_;
  DisconnectHandler on_disconnect_;
  Sink sink_;
  std::atomic<size_t> sent_to_local_{0}, sent_to_others_{0}, received_from_local_{0}, received_from_others_{0};
};

}  // namespace PS
