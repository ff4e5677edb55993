#include "executor.h"

#include "customer.h"
#include "postoffice.h"

namespace PS {

Executor::Executor(Customer& obj, Postoffice* sys) : obj_(obj), sys_(sys) {
  my_node_ = sys_->manager().van().my_node();
  for (const NodeID& id : {kServerGroup, kWorkerGroup, kCompGroup, kReplicaGroup, kOwnerGroup, kLiveGroup}) {
    Node n;
    n.role = Node::GROUP;
    n.id = id;
    nodes_[id].node = n;
  }
}

Executor::~Executor() { Stop(); }

void Executor::Start() {
  if (started_) return;
  started_ = true;
  thread_ = std::thread([this] { Run(); });
}

void Executor::Stop() {
  if (!started_) return;
  { Lock l(msg_mu_); done_ = true; }
  dag_cond_.notify_all();
  if (thread_.joinable()) thread_.join();
  started_ = false;
}

RemoteNode* Executor::GetRNode(const NodeID& id) {
  auto it = nodes_.find(id);
  return it == nodes_.end() ? nullptr : &it->second;
}

int Executor::NumAlive(const NodeID& id) {
  Lock l(node_mu_);
  RemoteNode* r = GetRNode(id);
  if (!r) return 0;
  if (r->node.role != Node::GROUP) return r->alive ? 1 : 0;
  int n = 0;
  for (auto* m : r->group) n += m->alive ? 1 : 0;
  return n;
}

bool Executor::CheckFinished(RemoteNode* rnode, int ts, bool sent) {
  if (ts < 0) return true;
  PS_CHECK(rnode != nullptr);
  auto done = [&](RemoteNode* r) {
    return !r->alive || (sent ? r->sent_req_tracker : r->recv_req_tracker).IsFinished(ts);
  };
  if (rnode->node.role == Node::GROUP) {
    for (auto* m : rnode->group) if (!done(m)) return false;
    return true;
  }
  return done(rnode);
}

int Executor::NumFinished(RemoteNode* rnode, int ts, bool sent) {
  if (ts < 0 || !rnode) return 0;
  auto done = [&](RemoteNode* r) { return (sent ? r->sent_req_tracker : r->recv_req_tracker).IsFinished(ts) ? 1 : 0; };
  if (rnode->node.role == Node::GROUP) {
    int n = 0;
    for (auto* m : rnode->group) n += done(m);
    return n;
  }
  return done(rnode);
}

void Executor::WaitSentReq(int ts) {
  ULock l(node_mu_);
  sent_req_cond_.wait(l, [this, ts] {
    auto it = sent_reqs_.find(ts);
    if (it == sent_reqs_.end()) return true;  // answered (entry retired) or never sent
    return false;
  });
}

void Executor::WaitRecvReq(int ts, const NodeID& sender) {
  ULock l(node_mu_);
  recv_req_cond_.wait(l, [this, ts, &sender] {
    RemoteNode* r = GetRNode(sender);
    return r != nullptr && CheckFinished(r, ts, false) &&
           // a group with no member yet has nothing to wait for only once nodes exist
           (r->node.role != Node::GROUP || !r->group.empty());
  });
}

void Executor::FinishRecvReq(int ts, const NodeID& sender) {
  {
    Lock l(node_mu_);
    RemoteNode* r = GetRNode(sender);
    PS_CHECK(r != nullptr) << "unknown node " << sender;
    if (r->node.role == Node::GROUP) for (auto* m : r->group) m->recv_req_tracker.Finish(ts);
    else r->recv_req_tracker.Finish(ts);
  }
  recv_req_cond_.notify_all();
  { Lock l(msg_mu_); }
  dag_cond_.notify_all();
}

int Executor::QueryRecvReq(int ts, const NodeID& sender) {
  Lock l(node_mu_);
  return NumFinished(GetRNode(sender), ts, false);
}

int Executor::Submit(Message* msg) {
  std::function<void()> run_now;
  int ts;
  {
    Lock l(node_mu_);
    Task& task = msg->task;
    PS_CHECK(!msg->recver.empty()) << "a request needs a recipient";
    ts = task.has_time ? task.time : time_ + 1;
    PS_CHECK_GE(ts, 0);
    task.set_time(ts);
    if (ts > time_) time_ = ts;
    task.request = true;
    task.customer_id = obj_.id();

    RemoteNode* rnode = GetRNode(msg->recver);
    PS_CHECK(rnode != nullptr) << my_node_.id << ": unknown recipient " << msg->recver;
    std::vector<RemoteNode*> dests;
    std::vector<Range<Key>> krs;
    if (rnode->node.role == Node::GROUP) {
      dests = rnode->group;
      krs = rnode->keys;
    } else {
      dests.push_back(rnode);
      Range<Key> kr = rnode->node.key;
      krs.push_back(kr.empty() ? Range<Key>::All() : kr);
    }
    size_t n = dests.size();
    std::vector<Message> parts(n);
    std::vector<Message*> ptrs(n);
    for (size_t i = 0; i < n; ++i) {
      parts[i].task = task;
      parts[i].recver = dests[i]->node.id;
      ptrs[i] = &parts[i];
    }
    if (n) obj_.Slice(*msg, krs, &ptrs);
    int num_sent = 0;
    sent_reqs_[ts] = ReqInfo{msg->recver, msg->callback};
    for (size_t i = 0; i < n; ++i) {
      RemoteNode* d = dests[i];
      Message& m = parts[i];
      m.recver = d->node.id;
      m.sender = my_node_.id;
      m.task.request = true;
      m.task.customer_id = obj_.id();
      m.task.set_time(ts);
      m.callback = nullptr;
      d->sent_req_tracker.Start(ts);
      if (!m.valid || !d->alive) {
        // nothing to send: this member counts as answered
        d->sent_req_tracker.Finish(ts);
        continue;
      }
      d->EncodeMessage(&m);
      ++num_sent;
      sys_->Queue(new Message(m));
    }
    if (num_sent == 0) {
      run_now = msg->callback;
      sent_reqs_.erase(ts);
    }
  }
  if (run_now) run_now();
  sent_req_cond_.notify_all();
  return ts;
}

void Executor::Reply(Message* request, Message* response) {
  Task& t = response->task;
  t.request = false;
  t.control = false;
  t.customer_id = obj_.id();
  t.set_time(request->task.time);
  response->recver = request->sender;
  response->sender = my_node_.id;
  request->replied = true;
  {
    Lock l(node_mu_);
    RemoteNode* r = GetRNode(response->recver);
    if (r == nullptr || !r->alive) return;
    r->EncodeMessage(response);
  }
  sys_->Queue(new Message(*response));
}

void Executor::Accept(Message* msg) {
  {
    Lock l(msg_mu_);
    recv_msgs_.push_back(std::shared_ptr<Message>(msg));
  }
  dag_cond_.notify_one();
}

void Executor::Run() {
  while (true) {
    {
      ULock l(msg_mu_);
      dag_cond_.wait(l, [this] { return done_ || PickActiveMsg(); });
      if (done_) break;
    }
    try {
      ProcessActiveMsg();
    } catch (const std::exception& e) {
      // an application error must not take the node's other customers down silently
      PS_LOG(ERROR) << my_node_.id << " customer " << obj_.id() << ": " << e.what();
      if (getenv("PSB_ABORT_ON_ERROR")) abort();
    }
  }
}

// msg_mu_ is held
bool Executor::PickActiveMsg() {
  Lock l(node_mu_);
  for (auto it = recv_msgs_.begin(); it != recv_msgs_.end();) {
    auto& msg = *it;
    RemoteNode* rnode = GetRNode(msg->sender);
    if (rnode == nullptr) { ++it; continue; }  // the sender is not registered here yet
    if (!rnode->alive) {
      PS_VLOG(1) << my_node_.id << ": drop a message from dead node " << msg->sender;
      it = recv_msgs_.erase(it);
      continue;
    }
    const bool req = msg->task.request;
    const int ts = msg->task.time;
    if ((req && rnode->recv_req_tracker.IsFinished(ts)) || (!req && rnode->sent_req_tracker.IsFinished(ts))) {
      PS_VLOG(1) << my_node_.id << ": drop a duplicate: " << msg->ShortDebugString();
      it = recv_msgs_.erase(it);
      continue;
    }
    bool ready = true;
    if (req) {
      for (int wt : msg->task.wait_time) {
        if (!rnode->recv_req_tracker.IsFinished(wt)) { ready = false; break; }
      }
    }
    if (ready) {
      active_msg_ = msg;
      recv_msgs_.erase(it);
      rnode->DecodeMessage(active_msg_.get());
      PS_VLOG(2) << my_node_.id << " picks " << active_msg_->ShortDebugString();
      return true;
    }
    ++it;
  }
  return false;
}

void Executor::ProcessActiveMsg() {
  std::shared_ptr<Message> msg = active_msg_;
  active_msg_.reset();
  const bool req = msg->task.request;
  const int ts = msg->task.time;
  const NodeID sender = msg->sender;
  if (req) {
    { Lock l(node_mu_); last_request_ = msg; }
    obj_.ProcessRequest(msg.get());
    if (msg->finished) {
      // the app did not defer completion: mark done and acknowledge
      FinishRecvReq(ts, sender);
      if (!msg->replied) obj_.Reply(msg.get());
    }
    return;
  }
  { Lock l(node_mu_); last_response_ = msg; }
  obj_.ProcessResponse(msg.get());
  std::function<void()> cb;
  bool all = false;
  {
    Lock l(node_mu_);
    RemoteNode* r = GetRNode(sender);
    if (r) r->sent_req_tracker.Finish(ts);
    auto it = sent_reqs_.find(ts);
    if (it != sent_reqs_.end()) {
      RemoteNode* orig = GetRNode(it->second.recver);
      all = orig == nullptr || CheckFinished(orig, ts, true);
      if (all) cb = std::move(it->second.callback);
    }
  }
  if (all) {
    // the callback completes before any Wait(ts) returns
    if (cb) cb();
    { Lock l(node_mu_); sent_reqs_.erase(ts); }
    sent_req_cond_.notify_all();
  }
}

void Executor::AddNode(const Node& node) {
  {
    Lock l(node_mu_);
    RemoteNode& r = nodes_[node.id];
    bool fresh = r.node.id.empty();
    if (!fresh) {
      for (const NodeID& g : {kServerGroup, kWorkerGroup, kCompGroup, kLiveGroup, kReplicaGroup, kOwnerGroup})
        nodes_[g].RemoveGroupNode(&r);
    }
    r.node = node;
    r.alive = true;
    if (node.role == Node::SERVER) { nodes_[kServerGroup].AddGroupNode(&r); nodes_[kCompGroup].AddGroupNode(&r); }
    if (node.role == Node::WORKER) { nodes_[kWorkerGroup].AddGroupNode(&r); nodes_[kCompGroup].AddGroupNode(&r); }
    nodes_[kLiveGroup].AddGroupNode(&r);
    // replica / owner groups of a server: the num_replicas_ servers whose ranges
    // precede / follow mine in the ring (chain replication layout)
    if (num_replicas_ > 0 && my_node_.role == Node::SERVER && node.role == Node::SERVER && node.id != my_node_.id) {
      nodes_[kReplicaGroup].AddGroupNode(&r);
      nodes_[kOwnerGroup].AddGroupNode(&r);
    }
    if (node.id == my_node_.id) my_node_ = node;
  }
  { Lock l(msg_mu_); }
  dag_cond_.notify_all();
  recv_req_cond_.notify_all();
}

void Executor::RemoveNode(const Node& node) {
  {
    Lock l(node_mu_);
    auto it = nodes_.find(node.id);
    if (it == nodes_.end()) return;
    RemoteNode& r = it->second;
    r.alive = false;
    for (const NodeID& g : {kServerGroup, kWorkerGroup, kCompGroup, kLiveGroup, kReplicaGroup, kOwnerGroup})
      nodes_[g].RemoveGroupNode(&r);
    // requests that were only waiting for this node are complete now
    std::vector<int> finished;
    for (auto& kv : sent_reqs_) {
      RemoteNode* orig = GetRNode(kv.second.recver);
      if (orig == nullptr || CheckFinished(orig, kv.first, true)) finished.push_back(kv.first);
    }
    for (int ts : finished) sent_reqs_.erase(ts);
  }
  sent_req_cond_.notify_all();
  recv_req_cond_.notify_all();
  { Lock l(msg_mu_); }
  dag_cond_.notify_all();
}

void Executor::ReplaceNode(const Node& old_node, const Node& new_node) {
  RemoveNode(old_node);
  AddNode(new_node);
}

}  // namespace PS
