// Postoffice: one per node. Owns the Manager (membership), the Van
// (transport), the outgoing queue with task packing, and the send / receive
// threads. Counterpart of system/postoffice.h:9-52, system/postoffice.cc:25-131.
// Unlike the reference it is an ordinary object, so several nodes can live in one
// process (in-process Van); `instance()` is the process default.
#pragma once
#include "env.h"
#include "manager.h"
#include "threading.h"
#include "van.h"

namespace PS {

class Postoffice {
 public:
  Postoffice();
  ~Postoffice();
  static Postoffice& instance() { static Postoffice po; return po; }

  // Joins the system and runs the app on the calling thread.
  void Run(const Options& opt);
  // Same, but returns once the node has joined (the app's Run() is not called).
  void Start(const Options& opt);
  void Stop();
  // Sends a message (takes ownership). Header-only requests carrying `more` are
  // packed into one wire message per (recipient, customer) until one without
  // `more` arrives. A message goes out on the calling thread when nothing is
  // waiting to be sent (a hand-over to the send thread costs more than writing a
  // small message to a socket); otherwise it joins the queue of the send thread,
  // so the messages of one thread leave in the order in which it queued them.
  void Queue(Message* msg);

  Manager& manager() { return manager_; }
  const Options& options() const { return opt_; }
  bool running() const { return running_; }

 private:
  void Send();
  void Dispatch(const MessagePtr& msg);   // queue it, or send it here and now
  void SendNow(Message* msg);
  void Recv();
  bool Incoming(Message* msg);            // unpacks packed tasks, then Process() for each; takes ownership
  bool Process(Message* msg);
  void StartThreads();
  void InstallSink();

  Options opt_;
  Manager manager_;
  ThreadsafeQueue<MessagePtr> sending_queue_;
  std::atomic<int> pending_sends_{0};     // messages in sending_queue_ or being sent by the send thread
  std::mutex send_mu_;                    // held by whoever is writing to the van
  std::mutex pack_mu_;
  std::map<std::pair<NodeID, int>, MessagePtr> pack_;
  std::thread recv_thread_, send_thread_;
  std::atomic<bool> running_{false};
  std::atomic<bool> sink_open_{true};     // false once the manager has said that the node is leaving
  PS_DISALLOW_COPY(Postoffice);
};

}  // namespace PS
