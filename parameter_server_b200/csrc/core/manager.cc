#include "manager.h"

#include <fstream>
#include <unistd.h>

#include "customer.h"
#include "postoffice.h"

namespace PS {

void Manager::StopCustomers() {
  // Join every customer's executor thread before any customer is destroyed: a
  // destructor must not run while the thread may still call into the object.
  std::vector<Customer*> all;
  {
    Lock l(customer_mu_);
    for (auto& c : customers_) all.push_back(c.second);
  }
  for (Customer* c : all) c->executor()->Stop();
}

Manager::~Manager() {
  StopCustomers();
  // the app is owned here unless an external factory keeps it
  if (!App::external_ownership()) delete app_;
  app_ = nullptr;
}

void Manager::Init(const Options& opt_in) {
  opt_ = opt_in;
  if (opt_.my_node.empty() || getenv("DMLC_PS_ROOT_URI")) opt_.InitFromEnv();
  Node me = Van::ParseNode(opt_.my_node);
  Node sch = Van::ParseNode(opt_.scheduler);
  van_.set_disconnect_handler([this](const NodeID& id) { NodeDisconnected(id); });
  van_.Init(me, sch, opt_.local);
  if (IsScheduler()) {
    node_assigner_.reset(new NodeAssigner(opt_.num_servers, Range<Key>(opt_.key_start, opt_.key_end)));
    // the application configuration: file content followed by the inline string
    std::string conf;
    if (!opt_.app_file.empty()) {
      std::ifstream in(opt_.app_file);
      PS_CHECK(in.good()) << "cannot read " << opt_.app_file;
      std::stringstream ss;
      ss << in.rdbuf();
      conf = ss.str();
    }
    conf += opt_.app_conf;
    app_conf_ = conf;
    Node self = my_node();
    node_assigner_->assign(&self);
    AddNode(self);
    CreateApp(conf);
    Lock l(nodes_mu_);
    is_my_node_inited_ = true;
  } else {
    // ask the scheduler for the application configuration
    Task task = NewControlTask(Control::REQUEST_APP);
    task.ctrl.node.push_back(my_node());
    SendTask(van_.scheduler(), task);
  }
}

void Manager::CreateApp(const std::string& conf) {
  app_ = App::Create(conf, sys_);
  PS_CHECK(app_ != nullptr) << "the application factory returned null";
}

void Manager::Run(bool run_app) {
  {
    ULock l(nodes_mu_);
    nodes_cv_.wait(l, [this] { return is_my_node_inited_ || done_; });
  }
  if (done_) return;
  if (van_.my_node().role == Node::WORKER) WaitServersReady();
  if (run_app && app_) app_->Run();
}

void Manager::Stop() {
  if (IsScheduler()) {
    // wait until every other node is ready to exit, then release them
    {
      ULock l(nodes_mu_);
      // A job that only the scheduler works on (model evaluation) can be over before the other nodes have
      // joined: they must still find the scheduler, register and be sent away properly, or they would
      // report a lost scheduler. Nodes that were lost on the way are not waited for.
      nodes_cv_.wait_for(l, std::chrono::seconds(30), [this] {
        return (num_servers_ >= opt_.num_servers && num_workers_ >= opt_.num_workers) || !failure_notified_.empty();
      });
      in_exit_ = true;
      nodes_cv_.wait_for(l, std::chrono::seconds(120), [this] { return num_active_nodes_ <= 1; });
    }
    Task task = NewControlTask(Control::EXIT);
    for (auto& n : nodes()) if (n.id != my_node().id) SendTask(n.id, task);
    std::this_thread::sleep_for(std::chrono::milliseconds(100));
    done_ = true;
  } else {
    Task task = NewControlTask(Control::READY_TO_EXIT);
    SendTask(van_.scheduler(), task);
    // idle until EXIT arrives
    ULock l(nodes_mu_);
    nodes_cv_.wait_for(l, std::chrono::seconds(120), [this] { return done_.load(); });
    done_ = true;
  }
}

Task Manager::NewControlTask(Control::Command cmd) {
  Task task;
  task.control = true;
  task.request = true;
  task.set_time(0);
  task.mutable_ctrl()->cmd = cmd;
  return task;
}

void Manager::SendTask(const NodeID& recver, const Task& task) {
  auto msg = new Message(task);
  msg->recver = recver;
  msg->sender = my_node().id;
  sys_->Queue(msg);
}

bool Manager::Process(Message* msg) {
  const Task& task = msg->task;
  PS_CHECK(task.control && task.has_ctrl);
  const Control& ctrl = task.ctrl;
  if (task.request) {
    switch (ctrl.cmd) {
      case Control::REQUEST_APP: {
        PS_CHECK(IsScheduler());
        PS_CHECK_EQ(ctrl.node.size(), (size_t)1);
        van_.Connect(ctrl.node[0]);
        Task reply;
        reply.control = true;
        reply.request = false;
        reply.set_time(task.time);
        reply.msg = app_conf_;
        reply.mutable_ctrl()->cmd = Control::REQUEST_APP;
        SendTask(ctrl.node[0].id, reply);
        break;
      }
      case Control::REGISTER_NODE: {
        PS_CHECK(IsScheduler());
        PS_CHECK_EQ(ctrl.node.size(), (size_t)1);
        Node node = ctrl.node[0];
        node_assigner_->assign(&node);
        AddNode(node);
        break;
      }
      case Control::REPORT_PERF: break;  // heartbeat reports are collected by the dashboard, if any
      case Control::READY_TO_EXIT: {
        PS_CHECK(IsScheduler());
        { Lock l(nodes_mu_); --num_active_nodes_; }
        nodes_cv_.notify_all();
        break;
      }
      case Control::ADD_NODE:
      case Control::UPDATE_NODE: {
        for (const auto& n : ctrl.node) AddNode(n);
        break;
      }
      case Control::REPLACE_NODE: {
        PS_CHECK_EQ(ctrl.node.size(), (size_t)2);
        RemoveNode(ctrl.node[0].id);
        AddNode(ctrl.node[1]);
        break;
      }
      case Control::REMOVE_NODE: {
        for (const auto& n : ctrl.node) RemoveNode(n.id);
        break;
      }
      case Control::EXIT: {
        done_ = true;
        nodes_cv_.notify_all();
        return false;
      }
      default: break;
    }
  } else {
    if (ctrl.cmd == Control::REQUEST_APP) {
      // the scheduler answered with the configuration: create the app, then register
      PS_CHECK(!IsScheduler());
      app_conf_ = task.msg;
      CreateApp(task.msg);
      Task reg = NewControlTask(Control::REGISTER_NODE);
      reg.ctrl.node.push_back(my_node());
      SendTask(van_.scheduler(), reg);
    }
  }
  return true;
}

void Manager::AddNode(const Node& node) {
  bool is_new;
  {
    Lock l(nodes_mu_);
    is_new = nodes_.find(node.id) == nodes_.end();
    nodes_[node.id] = node;
  }
  if (node.id == my_node().id) van_.UpdateMyNode(node);
  van_.Connect(node);
  {
    Lock l(customer_mu_);
    for (auto& c : customers_) c.second->executor()->AddNode(node);
  }
  if (is_new) {
    // Counted only now: WaitServersReady / WaitWorkersReady release an app that then submits to
    // the server or worker group, and the node must already be a member of every customer's groups.
    Lock l(nodes_mu_);
    if (node.role == Node::WORKER) ++num_workers_;
    if (node.role == Node::SERVER) ++num_servers_;
    ++num_active_nodes_;
  }
  if (IsScheduler() && node.id != my_node().id) {
    // the newcomer learns every node; everybody else learns the newcomer
    Task all = NewControlTask(Control::ADD_NODE);
    for (auto& n : nodes()) all.ctrl.node.push_back(n);
    SendTask(node.id, all);
    Task one = NewControlTask(Control::ADD_NODE);
    one.ctrl.node.push_back(node);
    for (auto& n : nodes()) {
      if (n.id == node.id || n.id == my_node().id) continue;
      SendTask(n.id, one);
    }
  }
  if (node.id == my_node().id && !IsScheduler()) {
    Lock l(nodes_mu_);
    is_my_node_inited_ = true;
  }
  nodes_cv_.notify_all();
  PS_VLOG(1) << my_node().id << " adds node " << node.ShortDebugString();
}

void Manager::RemoveNode(const NodeID& node_id) {
  Node node;
  {
    Lock l(nodes_mu_);
    auto it = nodes_.find(node_id);
    if (it == nodes_.end()) return;
    node = it->second;
    if (node.role == Node::WORKER) --num_workers_;
    if (node.role == Node::SERVER) --num_servers_;
    --num_active_nodes_;
    nodes_.erase(it);
  }
  {
    Lock l(customer_mu_);
    for (auto& c : customers_) c.second->executor()->RemoveNode(node);
  }
  if (node_assigner_) node_assigner_->remove(node);
  if (!IsScheduler()) {
    // A node that did not see the connection drop itself learns of the loss from the scheduler's
    // REMOVE_NODE: its failure handlers run once per lost node, whichever way the news came.
    std::vector<NodeFailureHandler> hs;
    {
      Lock l(nodes_mu_);
      if (failure_notified_.insert(node_id).second) hs = node_failure_handlers_;
    }
    for (auto& h : hs) h(node_id);
  }
  if (IsScheduler()) {
    Task task = NewControlTask(Control::REMOVE_NODE);
    task.ctrl.node.push_back(node);
    for (auto& n : nodes()) if (n.id != my_node().id) SendTask(n.id, task);
  }
  nodes_cv_.notify_all();
  PS_VLOG(1) << my_node().id << " removes node " << node_id;
}

void Manager::NodeDisconnected(const NodeID& node_id) {
  if (done_ || in_exit_) return;
  std::vector<NodeFailureHandler> hs;
  {
    Lock l(nodes_mu_);
    if (nodes_.find(node_id) == nodes_.end() && node_id != van_.scheduler().id) return;
    if (failure_notified_.insert(node_id).second) hs = node_failure_handlers_;
  }
  PS_LOG(WARN) << my_node().id << ": node " << node_id << " is disconnected";
  for (auto& h : hs) h(node_id);
  if (IsScheduler()) {
    RemoveNode(node_id);
  } else if (node_id == van_.scheduler().id) {
    // nothing can make progress without the scheduler
    PS_LOG(ERROR) << my_node().id << ": the scheduler is gone";
    done_ = true;
    nodes_cv_.notify_all();
    if (opt_.exit_on_scheduler_loss) {
      std::this_thread::sleep_for(std::chrono::seconds(1));
      _exit(1);
    }
  }
}

void Manager::AddCustomer(Customer* obj) {
  {
    Lock l(customer_mu_);
    PS_CHECK_EQ(customers_.count(obj->id()), (size_t)0) << "customer id " << obj->id() << " already exists";
    customers_[obj->id()] = obj;
  }
  for (auto& n : nodes()) obj->executor()->AddNode(n);
  customer_cv_.notify_all();
}

void Manager::RemoveCustomer(int id) {
  Lock l(customer_mu_);
  customers_.erase(id);
}

Customer* Manager::customer(int id) {
  ULock l(customer_mu_);
  customer_cv_.wait_for(l, std::chrono::seconds(10), [this, id] { return customers_.count(id) > 0; });
  auto it = customers_.find(id);
  return it == customers_.end() ? nullptr : it->second;
}

int Manager::NextCustomerID() {
  Lock l(customer_mu_);
  while (customers_.count(next_customer_id_)) ++next_customer_id_;
  return next_customer_id_++;
}

void Manager::WaitServersReady() {
  ULock l(nodes_mu_);
  nodes_cv_.wait(l, [this] { return num_servers_ >= opt_.num_servers || done_; });
}

void Manager::WaitWorkersReady() {
  ULock l(nodes_mu_);
  nodes_cv_.wait(l, [this] { return num_workers_ >= opt_.num_workers || done_; });
}

}  // namespace PS
