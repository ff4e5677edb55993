#include "learner.h"

namespace PS {

void ISGDScheduler::Run() {
  // merge progress per sender, print about once a second
  monitor_.set_merger([](const SGDProgress& src, SGDProgress* dst) {
    dst->objective.insert(dst->objective.end(), src.objective.begin(), src.objective.end());
    dst->accuracy.insert(dst->accuracy.end(), src.accuracy.begin(), src.accuracy.end());
    dst->auc.insert(dst->auc.end(), src.auc.begin(), src.auc.end());
    dst->num_examples_processed += src.num_examples_processed;
    if (src.nnz || src.weight_sum || src.delta_sum) {
      dst->nnz = src.nnz;
      dst->weight_sum += src.weight_sum;
      dst->delta_sum += src.delta_sum;
    }
  });
  monitor_.set_printer(1.0, [this](double t, std::unordered_map<NodeID, SGDProgress>* p) {
    std::string line = ProgressLine(t, p);
    if (show_progress_) {
      if (!printed_header_) { PS_NOTICE("%s", ProgressHeader().c_str()); printed_header_ = true; }
      PS_NOTICE("%s", line.c_str());
    }
  });
  // a dead worker's files go back into the pool
  sys_->manager().AddNodeFailureHandler([this](const NodeID& id) { if (workload_pool_) workload_pool_->restore(id); });
  PS_CHECK(workload_pool_ != nullptr);
  sys_->manager().WaitServersReady();
  sys_->manager().WaitWorkersReady();
  workload_pool_->waitUtilDone();
  // ask the servers to save the model
  Task save;
  save.mutable_sgd()->cmd = SGDCall::SAVE_MODEL;
  int ts = Submit(save, kServerGroup);
  Wait(ts);
}

void LockstepSGDScheduler::Grant(bool final_round) {
  Task t;
  {
    Lock l(lease_mu_);
    if (final_sent_) return;
    if (final_round) {
      final_sent_ = true;                       // the limit in force is the last round of the job
    } else {
      const uint64_t want = max_round_ + lease_;
      if (limit_ != 0 && want < limit_ + lease_ / 4) return;   // still far enough ahead
      limit_ = want;
    }
    t.mutable_sgd()->cmd = SGDCall::ROUND_LIMIT;
    t.sgd.round_limit = (int64_t)limit_;
    t.sgd.final_round = final_round;
  }
  int ts = Submit(t, kWorkerGroup);
  if (final_round) Wait(ts);                    // a worker answers once its last round has completed
}

void LockstepSGDScheduler::Run() {
  monitor_.set_merger([this](const SGDProgress& src, SGDProgress* dst) {
    dst->objective.insert(dst->objective.end(), src.objective.begin(), src.objective.end());
    dst->accuracy.insert(dst->accuracy.end(), src.accuracy.begin(), src.accuracy.end());
    dst->auc.insert(dst->auc.end(), src.auc.begin(), src.auc.end());
    dst->num_examples_processed += src.num_examples_processed;
    if (src.nnz || src.weight_sum || src.delta_sum) {
      dst->nnz = src.nnz;
      dst->weight_sum += src.weight_sum;
      dst->delta_sum += src.delta_sum;
    }
    bool ahead = false;
    {
      Lock l(lease_mu_);
      if (src.round > max_round_) { max_round_ = src.round; ahead = true; }
    }
    if (ahead) Grant(false);
  });
  monitor_.set_printer(1.0, [this](double t, std::unordered_map<NodeID, SGDProgress>* p) {
    std::string line = ProgressLine(t, p);
    if (show_progress_) {
      if (!printed_header_) { PS_NOTICE("%s", ProgressHeader().c_str()); printed_header_ = true; }
      PS_NOTICE("%s", line.c_str());
    }
  });
  sys_->manager().AddNodeFailureHandler([this](const NodeID& id) { NodeLost(id); });
  sys_->manager().WaitServersReady();
  sys_->manager().WaitWorkersReady();
  Grant(false);                                 // the first lease
  pool_.waitUtilDone();
  Grant(true);
  Task save;
  save.mutable_sgd()->cmd = SGDCall::SAVE_MODEL;
  int ts = Submit(save, kServerGroup);
  Wait(ts);
}

void ISGDScheduler::ProcessRequest(Message* request) {
  if (request->task.has_sgd && request->task.sgd.cmd == SGDCall::REQUEST_WORKLOAD) {
    SendWorkload(request->sender);
  }
}

void ISGDScheduler::ProcessResponse(Message* response) {
  const Task& t = response->task;
  if (t.has_sgd && t.sgd.cmd == SGDCall::UPDATE_MODEL) {
    // the worker finished a workload: mark it and hand out the next one
    for (int id : t.sgd.load.id) workload_pool_->finish(id);
    SendWorkload(response->sender);
  }
}

bool ISGDScheduler::SendWorkload(const NodeID& recver) {
  Task task;
  task.mutable_sgd()->cmd = SGDCall::UPDATE_MODEL;
  if (!workload_pool_->assign(recver, &task.sgd.load)) return false;
  task.sgd.has_load = true;
  Submit(task, recver);
  return true;
}

bool LockstepSGDScheduler::SendWorkload(const NodeID& recver) {
  const bool sent = ISGDScheduler::SendWorkload(recver);
  Lock l(idle_mu_);
  if (sent) idle_.erase(recver); else idle_.insert(recver);
  return sent;
}

void LockstepSGDScheduler::NodeLost(const NodeID& id) {
  pool_.restore(id);
  std::vector<NodeID> waiting;
  {
    Lock l(idle_mu_);
    idle_.erase(id);
    waiting.assign(idle_.begin(), idle_.end());
  }
  // workers that found the pool empty earlier will not ask again by themselves
  for (const NodeID& w : waiting) SendWorkload(w);
}

std::string ISGDScheduler::ProgressHeader() {
  return " sec  examples    loss      auc   accuracy   |w|_0  updt ratio";
}

std::string ISGDScheduler::ProgressLine(double time, std::unordered_map<NodeID, SGDProgress>* progress) {
  uint64_t num_ex = 0, nnz_w = 0;
  double w_sum = 0, delta_sum = 0;
  std::vector<double> objv, auc, acc;
  for (auto& it : *progress) {
    SGDProgress& p = it.second;
    num_ex += p.num_examples_processed;
    nnz_w += p.nnz;
    w_sum += p.weight_sum;
    delta_sum += p.delta_sum;
    objv.insert(objv.end(), p.objective.begin(), p.objective.end());
    auc.insert(auc.end(), p.auc.begin(), p.auc.end());
    acc.insert(acc.end(), p.accuracy.begin(), p.accuracy.end());
    // counters are per report interval
    p.objective.clear(); p.auc.clear(); p.accuracy.clear();
    p.num_examples_processed = 0; p.weight_sum = 0; p.delta_sum = 0;
  }
  num_ex_processed_ += num_ex;
  auto mean = [](const std::vector<double>& v) { double s = 0; for (double x : v) s += x; return v.empty() ? 0 : s / v.size(); };
  double objv_sum = 0;
  for (double o : objv) objv_sum += o;
  std::ostringstream ss;
  ss << std::setw(4) << (int)time << "  " << std::scientific << std::setprecision(2) << (double)num_ex_processed_.load()
     << "  " << std::setprecision(3) << (num_ex ? objv_sum / num_ex : 0.0) << "  " << std::fixed << std::setprecision(4)
     << mean(auc) << "  " << mean(acc) << "  " << std::scientific << std::setprecision(2) << (double)nnz_w << "  "
     << (w_sum > 0 ? std::sqrt(delta_sum) / std::sqrt(w_sum) : 0.0);
  return ss.str();
}

}  // namespace PS
