#include "postoffice.h"

#include "customer.h"
#include "data.h"

namespace PS {

namespace {
// set on a thread that must not write to sockets itself: the van's poll thread while it runs the sink (if it
// blocked on a peer whose poll thread is blocked on this node, neither would read again)
thread_local bool tl_queue_only = false;
}  // namespace

Postoffice::Postoffice() : manager_(this) {}

Postoffice::~Postoffice() {
  manager_.StopCustomers();
  if (running_) {
    running_ = false;
    auto t = std::make_shared<Message>();
    t->terminate = true;
    sending_queue_.push(t);
    manager_.van().WakeUp();
  }
  if (send_thread_.joinable()) send_thread_.join();
  if (recv_thread_.joinable()) recv_thread_.join();
}

void Postoffice::InstallSink() {
  // over sockets the van's poll thread runs the receive path itself; the receive thread then only waits for
  // the end (in-process nodes have no poll thread: their receive thread takes messages from the peer's push)
  manager_.van().set_sink([this](const MessagePtr& m) {
    if (!sink_open_) return;
    tl_queue_only = true;
    auto* copy = new Message(*m);
    copy->recver = manager_.van().my_node().id;
    if (!Incoming(copy)) sink_open_ = false;
  });
}

void Postoffice::StartThreads() {
  ReaderFlags& rf = ReaderFlags::get();
  if (opt_.hash_kernel) rf.hash_kernel = opt_.hash_kernel;
  if (opt_.shuffle_fea_id) rf.shuffle_fea_id = true;
  if (opt_.line_limit > 0) rf.line_limit = opt_.line_limit;
  if (opt_.num_threads > 0) rf.parse_threads = opt_.num_threads;
  running_ = true;
  manager_.van().enable_sink();
  recv_thread_ = std::thread([this] { Recv(); });
  send_thread_ = std::thread([this] { Send(); });
}

void Postoffice::Run(const Options& opt) {
  opt_ = opt;
  InstallSink();
  manager_.Init(opt);
  StartThreads();
  manager_.Run(true);
}

void Postoffice::Start(const Options& opt) {
  opt_ = opt;
  InstallSink();
  manager_.Init(opt);
  StartThreads();
  manager_.Run(false);
}

void Postoffice::Stop() {
  manager_.Stop();
  // no customer thread may still be replying (and queueing messages) while the
  // send thread and the queues go away
  manager_.StopCustomers();
  if (running_) {
    running_ = false;
    auto t = std::make_shared<Message>();
    t->terminate = true;
    sending_queue_.push(t);
    manager_.van().WakeUp();
  }
  if (send_thread_.joinable()) send_thread_.join();
  if (recv_thread_.joinable()) recv_thread_.join();
  PS_VLOG(1) << manager_.van().Statistic();
  manager_.van().Destroy();
}

void Postoffice::SendNow(Message* msg) {
  size_t bytes = 0;
  manager_.van().Send(msg, &bytes);
  if (msg->task.request) manager_.AddRequest(msg);
}

void Postoffice::Send() {
  while (true) {
    MessagePtr msg;
    sending_queue_.wait_and_pop(msg);
    if (msg->terminate) break;
    {
      Lock l(send_mu_);
      SendNow(msg.get());
    }
    --pending_sends_;
  }
}

void Postoffice::Dispatch(const MessagePtr& msg) {
  // Nothing queued and nobody sending: this thread writes the message itself. A message that another
  // thread queues in the meantime is not ordered against this one anyway; this thread's own earlier
  // messages have left (they were sent here) or are still pending (then this one queues up behind them).
  // Only what cannot make this thread wait for the peer: submitting threads hold their executor's lock, and a
  // thread that held it while blocked in a write would stall the node's whole receive path (two nodes doing so
  // to each other would never read again). Large payloads go through the send thread, which holds no such lock.
  size_t payload = msg->key.size() + 512;
  for (auto& v : msg->value) payload += v.size();
  if (running_ && !tl_queue_only && pending_sends_.load() == 0 && send_mu_.try_lock()) {
    if (pending_sends_.load() == 0 && manager_.van().WritableNow(msg->recver, payload)) {
      SendNow(msg.get());
      send_mu_.unlock();
      return;
    }
    send_mu_.unlock();
  }
  ++pending_sends_;
  sending_queue_.push(msg);
}

void Postoffice::Queue(Message* raw) {
  MessagePtr msg(raw);
  const Task& t = msg->task;
  const bool header_only = !msg->has_key() && msg->value.empty();
  if (!t.control && t.request && header_only) {
    // task packing
    auto key = std::make_pair(msg->recver, t.customer_id);
    Lock l(pack_mu_);
    auto it = pack_.find(key);
    if (t.more) {
      if (it == pack_.end()) {
        auto holder = std::make_shared<Message>();
        holder->recver = msg->recver;
        holder->sender = msg->sender;
        holder->task.request = true;
        holder->task.customer_id = t.customer_id;
        holder->task.more = true;
        it = pack_.emplace(key, holder).first;
      }
      it->second->task.task.push_back(t);
      return;
    }
    if (it != pack_.end()) {
      // flush: the pack plus this closing task travel as one wire message
      MessagePtr holder = it->second;
      pack_.erase(it);
      holder->task.task.push_back(t);
      Dispatch(holder);
      return;
    }
  }
  Dispatch(msg);
}

void Postoffice::Recv() {
  while (true) {
    auto msg = new Message();
    size_t bytes = 0;
    if (!manager_.van().Recv(msg, &bytes)) { delete msg; break; }
    if (!Incoming(msg)) break;
  }
}

bool Postoffice::Incoming(Message* msg) {
  if (!msg->task.control && msg->task.request && !msg->task.task.empty() && msg->task.more) {
    // unpack
    std::vector<Task> tasks = msg->task.task;
    for (auto& t : tasks) {
      auto unpacked = new Message(t);
      unpacked->sender = msg->sender;
      unpacked->recver = msg->recver;
      if (!Process(unpacked)) { delete msg; return false; }
    }
    delete msg;
    return true;
  }
  return Process(msg);
}

bool Postoffice::Process(Message* msg) {
  if (!msg->task.request) manager_.AddResponse(msg);
  if (msg->task.control) {
    bool keep_going = manager_.Process(msg);
    delete msg;
    return keep_going;
  }
  Customer* c = manager_.customer(msg->task.customer_id);
  if (c == nullptr) {
    PS_LOG(WARN) << manager_.van().my_node().id << ": no customer " << msg->task.customer_id << ", dropping "
                 << msg->ShortDebugString();
    delete msg;
    return true;
  }
  c->executor()->Accept(msg);  // takes ownership
  return true;
}

}  // namespace PS
