// Progress monitor (slaves report a progress record to the scheduler, which
// merges per sender and prints at most every `interval` seconds), heartbeat
// sampling, dashboard table and the task tracker.
// Counterparts: system/monitor.h:17-97, system/heartbeat_info.h:8-88 (+ .cc),
// system/proto/heartbeat.proto:3-31, system/dashboard.h:12-22 (+ .cc),
// system/task_tracker.h:11-55.
#pragma once
#include <fstream>
#include <iomanip>
#include "customer.h"
#include "postoffice.h"

namespace PS {

// P must provide std::string Serialize() const and bool Parse(const std::string&).
template <typename P>
class MonitorMaster : public Customer {
 public:
  explicit MonitorMaster(int id, Postoffice* po = nullptr) : Customer(id, po) {}
  typedef std::function<void(double time, std::unordered_map<NodeID, P>*)> Printer;
  typedef std::function<void(const P& src, P* dst)> Merger;
  // print at most once every `interval` seconds
  void set_printer(double interval, Printer p) { Lock l(mu_); interval_ = interval; printer_ = p; }
  void set_merger(Merger m) { Lock l(mu_); merger_ = m; }
  std::unordered_map<NodeID, P> progress() { Lock l(mu_); return progress_; }

  void ProcessRequest(Message* request) override {
    P prog;
    PS_CHECK(prog.Parse(request->task.msg));
    Lock l(mu_);
    if (merger_) merger_(prog, &progress_[request->sender]);
    else progress_[request->sender] = prog;
    double now = NowSeconds();
    if (start_ == 0) start_ = now;
    if (printer_ && now - last_print_ >= interval_) {
      last_print_ = now;
      printer_(now - start_, &progress_);
    }
  }
 private:
  std::unordered_map<NodeID, P> progress_;
  double interval_ = 1, last_print_ = 0, start_ = 0;
  Merger merger_;
  Printer printer_;
  std::mutex mu_;
};

template <typename P>
class MonitorSlaver : public Customer {
 public:
  MonitorSlaver(const NodeID& master, int id, Postoffice* po = nullptr) : Customer(id, po), master_(master) {}
  void Report(const P& prog) {
    Task report;
    report.msg = prog.Serialize();
    Submit(report, master_);
  }
 protected:
  NodeID master_;
};

// ---------------------------------------------------------------- heartbeat
struct HeartbeatReport {
  int32_t task_id = 0;
  std::string hostname;
  uint32_t seconds_since_epoch = 0;
  uint32_t total_time_milli = 0, busy_time_milli = 0;
  uint32_t net_in_mb = 0, net_out_mb = 0;
  uint32_t process_cpu_usage = 0, host_cpu_usage = 0;
  uint32_t process_rss_mb = 0, process_virt_mb = 0;
  uint32_t host_in_use_gb = 0, host_in_use_percentage = 0;
  uint32_t host_net_in_bw = 0, host_net_out_bw = 0;
  std::string Serialize() const {
    Writer w;
    w.I64(task_id); w.Str(hostname);
    for (uint32_t v : {seconds_since_epoch, total_time_milli, busy_time_milli, net_in_mb, net_out_mb,
                       process_cpu_usage, host_cpu_usage, process_rss_mb, process_virt_mb, host_in_use_gb,
                       host_in_use_percentage, host_net_in_bw, host_net_out_bw}) w.U64(v);
    return w.str();
  }
  bool Parse(const std::string& s) {
    Reader r(s.data(), s.size());
    task_id = (int32_t)r.I64(); hostname = r.Str();
    for (uint32_t* v : {&seconds_since_epoch, &total_time_milli, &busy_time_milli, &net_in_mb, &net_out_mb,
                        &process_cpu_usage, &host_cpu_usage, &process_rss_mb, &process_virt_mb, &host_in_use_gb,
                        &host_in_use_percentage, &host_net_in_bw, &host_net_out_bw}) *v = (uint32_t)r.U64();
    return r.ok();
  }
};

// Samples /proc counters between successive get() calls.
class HeartbeatInfo {
 public:
  enum class TimerType : size_t { BUSY = 0, NUM };
  HeartbeatInfo() { start_ = NowSeconds(); last_ = Sample(); }
  void startTimer(TimerType t) { Lock l(mu_); timer_start_[(size_t)t] = NowSeconds(); }
  void stopTimer(TimerType t) {
    Lock l(mu_);
    timer_total_[(size_t)t] += NowSeconds() - timer_start_[(size_t)t];
  }
  void increaseInBytes(size_t d) { in_bytes_ += d; }
  void increaseOutBytes(size_t d) { out_bytes_ += d; }
  void init(const std::string& interface, const std::string& hostname) { interface_ = interface; hostname_ = hostname; }
  HeartbeatReport get() {
    Lock l(mu_);
    Snapshot now = Sample();
    HeartbeatReport r;
    r.hostname = hostname_;
    r.seconds_since_epoch = (uint32_t)time(nullptr);
    r.total_time_milli = (uint32_t)((now.t - last_.t) * 1e3);
    r.busy_time_milli = (uint32_t)(timer_total_[0] * 1e3);
    timer_total_[0] = 0;
    r.net_in_mb = (uint32_t)(in_bytes_.exchange(0) >> 20);
    r.net_out_mb = (uint32_t)(out_bytes_.exchange(0) >> 20);
    double dt_ticks = std::max<double>(1, (double)(now.host_total - last_.host_total));
    r.process_cpu_usage = (uint32_t)(100.0 * ncpu_ * (now.proc_ticks - last_.proc_ticks) / dt_ticks);
    r.host_cpu_usage = (uint32_t)(100.0 * ncpu_ * (now.host_busy - last_.host_busy) / dt_ticks);
    r.process_rss_mb = (uint32_t)(now.rss_kb >> 10);
    r.process_virt_mb = (uint32_t)(now.virt_kb >> 10);
    r.host_in_use_gb = (uint32_t)(now.mem_used_kb >> 20);
    r.host_in_use_percentage = now.mem_total_kb ? (uint32_t)(100 * now.mem_used_kb / now.mem_total_kb) : 0;
    double dt = std::max(1e-3, now.t - last_.t);
    r.host_net_in_bw = (uint32_t)((now.net_in - last_.net_in) / dt / (1 << 20));
    r.host_net_out_bw = (uint32_t)((now.net_out - last_.net_out) / dt / (1 << 20));
    last_ = now;
    return r;
  }
 private:
  struct Snapshot {
    double t = 0;
    uint64_t proc_ticks = 0, host_total = 0, host_busy = 0, rss_kb = 0, virt_kb = 0;
    uint64_t mem_total_kb = 0, mem_used_kb = 0, net_in = 0, net_out = 0;
  };
  Snapshot Sample() {
    Snapshot s;
    s.t = NowSeconds();
    { std::ifstream f("/proc/self/stat"); std::string tok; std::vector<std::string> v;
      while (f >> tok) v.push_back(tok);
      if (v.size() > 23) { s.proc_ticks = strtoull(v[13].c_str(), 0, 10) + strtoull(v[14].c_str(), 0, 10);
                           s.virt_kb = strtoull(v[22].c_str(), 0, 10) >> 10; s.rss_kb = strtoull(v[23].c_str(), 0, 10) * 4; } }
    { std::ifstream f("/proc/stat"); std::string cpu; uint64_t a[8] = {0};
      if (f >> cpu) { for (auto& x : a) f >> x; for (auto x : a) s.host_total += x; s.host_busy = s.host_total - a[3] - a[4]; } }
    { std::ifstream f("/proc/meminfo"); std::string k; uint64_t v; std::string unit; uint64_t avail = 0;
      while (f >> k >> v >> unit) { if (k == "MemTotal:") s.mem_total_kb = v; if (k == "MemAvailable:") avail = v; }
      s.mem_used_kb = s.mem_total_kb - avail; }
    { std::ifstream f("/proc/net/dev"); std::string line;
      while (std::getline(f, line)) {
        size_t c = line.find(':'); if (c == std::string::npos) continue;
        std::string name = line.substr(0, c); name.erase(0, name.find_first_not_of(' '));
        if (!interface_.empty() && name != interface_) continue;
        if (interface_.empty() && name == "lo") continue;
        std::istringstream ss(line.substr(c + 1)); uint64_t v[16] = {0};
        for (auto& x : v) ss >> x;
        s.net_in += v[0]; s.net_out += v[8];
      } }
    return s;
  }
  std::mutex mu_;
  std::string interface_, hostname_;
  double start_ = 0;
  int ncpu_ = (int)std::max(1u, std::thread::hardware_concurrency());
  double timer_start_[1] = {0}, timer_total_[1] = {0};
  std::atomic<size_t> in_bytes_{0}, out_bytes_{0};
  Snapshot last_;
};

// Table of the latest heartbeat of every node, ordered scheduler, servers, workers.
class Dashboard {
 public:
  void addTask(const NodeID& node, int task_id) { Lock l(mu_); data_[node].task_id = task_id; }
  void addReport(const NodeID& node, const std::string& report) {
    HeartbeatReport r;
    if (!r.Parse(report)) return;
    Lock l(mu_);
    int task = data_[node].task_id;
    data_[node] = r;
    data_[node].task_id = task;
  }
  std::string title() const {
    std::ostringstream ss;
    ss << std::setw(12) << "node" << std::setw(8) << "task" << std::setw(10) << "busy(ms)" << std::setw(10)
       << "in(MB)" << std::setw(10) << "out(MB)" << std::setw(8) << "cpu%" << std::setw(10) << "rss(MB)"
       << std::setw(10) << "host cpu%" << std::setw(12) << "host mem%";
    return ss.str();
  }
  std::string report() {
    Lock l(mu_);
    std::vector<NodeID> ids;
    for (auto& d : data_) ids.push_back(d.first);
    auto rank = [](const NodeID& id) { return id.empty() ? 3 : id[0] == 'H' ? 0 : id[0] == 'S' ? 1 : 2; };
    std::sort(ids.begin(), ids.end(), [&](const NodeID& a, const NodeID& b) {
      return rank(a) != rank(b) ? rank(a) < rank(b) : (a.size() != b.size() ? a.size() < b.size() : a < b);
    });
    std::ostringstream ss;
    ss << title() << "\n";
    for (auto& id : ids) {
      auto& r = data_[id];
      ss << std::setw(12) << id << std::setw(8) << r.task_id << std::setw(10) << r.busy_time_milli << std::setw(10)
         << r.net_in_mb << std::setw(10) << r.net_out_mb << std::setw(8) << r.process_cpu_usage << std::setw(10)
         << r.process_rss_mb << std::setw(10) << r.host_cpu_usage << std::setw(12) << r.host_in_use_percentage << "\n";
    }
    return ss.str();
  }
 private:
  std::mutex mu_;
  std::map<NodeID, HeartbeatReport> data_;
};

// id -> started/finished, with a blocking wait.
class TaskTracker {
 public:
  void wait(int id) { ULock l(mu_); cond_.wait(l, [this, id] { auto it = task_.find(id); return it != task_.end() && it->second; }); }
  void start(int id) { Lock l(mu_); task_[id] = false; }
  void finish(int id) { { Lock l(mu_); task_[id] = true; } cond_.notify_all(); }
  bool hasFinished(int id) { Lock l(mu_); auto it = task_.find(id); return it != task_.end() && it->second; }
  bool wasStarted(int id) { Lock l(mu_); return task_.count(id) > 0; }
 private:
  std::mutex mu_;
  std::condition_variable cond_;
  std::map<int, bool> task_;
};

}  // namespace PS
