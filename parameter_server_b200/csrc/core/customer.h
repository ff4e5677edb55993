// Customer: base class of every distributed object. Objects constructed with
// the same integer id on different nodes are the same logical object; they talk
// by submitting request messages with timestamps and dependencies, executed by
// the object's Executor. App is the per-node application object.
// Counterpart of system/customer.h:43-278.
#pragma once
#include "executor.h"
#include "message.h"

namespace PS {

class Postoffice;

class Customer {
 public:
  // `po` = the node this object lives on (default: the process-wide Postoffice)
  explicit Customer(int id, Postoffice* po = nullptr);
  virtual ~Customer();

  // ---- as a sender ----
  // Sends a header-only request to `recver` (a node id or a group id); returns its timestamp.
  int Submit(const Task& request, const NodeID& recver) {
    Message msg(request);
    msg.recver = recver;
    return Submit(&msg);
  }
  // Sends a request with payload; msg->callback (if set) runs once all recipients answered.
  int Submit(Message* request) { return exec_.Submit(request); }
  // Blocks until the request `timestamp` has been answered by every live recipient.
  void Wait(int timestamp) { exec_.WaitSentReq(timestamp); }
  // Splits `request` into one message per key range (one per member of the
  // recipient group). Default: every member gets a copy.
  virtual void Slice(const Message& request, const std::vector<Range<Key>>& krs, std::vector<Message*>* msgs) {
    for (auto m : *msgs) { NodeID recver = m->recver; *m = request; m->recver = recver; m->callback = nullptr; }
  }
  virtual void ProcessResponse(Message* response) {}
  std::shared_ptr<Message> LastResponse() { return exec_.last_response(); }

  // ---- as a receiver ----
  virtual void ProcessRequest(Message* request) {}
  std::shared_ptr<Message> LastRequest() { return exec_.last_request(); }
  // Blocks until the request `timestamp` from `sender` (node or group) is finished.
  void WaitReceivedRequest(int timestamp, const NodeID& sender) { exec_.WaitRecvReq(timestamp, sender); }
  // Marks `timestamp` of `sender` finished; a *virtual* timestamp (one nobody
  // sent) releases requests that depend on it.
  void FinishReceivedRequest(int timestamp, const NodeID& sender) { exec_.FinishRecvReq(timestamp, sender); }
  int NumDoneReceivedRequest(int timestamp, const NodeID& sender) { return exec_.QueryRecvReq(timestamp, sender); }
  void Reply(Message* request, Task response = Task()) {
    Message m(response);
    Reply(request, &m);
  }
  void Reply(Message* request, Message* response) { exec_.Reply(request, response); }

  int id() const { return id_; }
  Executor* executor() { return &exec_; }
  Postoffice& sys() { return *sys_; }

 protected:
  Postoffice* sys_;
  int id_;
  Executor exec_;
 private:
  PS_DISALLOW_COPY(Customer);
};

// The application object of a node; created on every node from the same
// configuration string by a registered factory.
class App : public Customer {
 public:
  explicit App(Postoffice* po = nullptr, int id = 0) : Customer(id, po) {}
  virtual ~App() {}
  typedef std::function<App*(const std::string& conf, Postoffice* po)> Factory;
  static void SetFactory(Factory f) { factory() = std::move(f); }
  static App* Create(const std::string& conf, Postoffice* po = nullptr) {
    PS_CHECK(factory()) << "no application factory registered";
    return factory()(conf, po);
  }
  // Runs on the main thread once the node has joined.
  virtual void Run();
  // true when app objects are owned by someone else (e.g. a Python factory):
  // the node's Manager then does not delete them
  static bool& external_ownership() { static bool v = false; return v; }
 private:
  static Factory& factory() { static Factory f; return f; }
};

}  // namespace PS
