// Per-peer state held by an Executor: liveness, which timestamps have been
// sent/received and finished, group membership ordered by key range, and the
// peer's own filter instances (so key-cache state is per peer).
// Counterpart of system/remote_node.h:13-65, system/remote_node.cc:7-56.
#pragma once
#include "filter.h"

namespace PS {

// Tracks which integer timestamps are finished.
class RequestTracker {
 public:
  void Start(int ts) { Set(ts, false); }
  void Finish(int ts) { Set(ts, true); }
  bool IsFinished(int ts) const { return ts < 0 || ((int)data_.size() > ts && data_[ts]); }
 private:
  void Set(int ts, bool v) {
    PS_CHECK_GE(ts, 0);
    PS_CHECK_LT(ts, 100000000);
    if ((int)data_.size() <= ts) data_.resize(ts * 2 + 5, false);
    data_[ts] = v;
  }
  std::vector<bool> data_;
};

struct RemoteNode {
  RemoteNode() {}
  ~RemoteNode() { for (auto& f : filters) delete f.second; }
  void EncodeMessage(Message* msg) {
    for (auto& conf : msg->task.filter) FindFilterOrCreate(conf)->encode(msg);
  }
  void DecodeMessage(Message* msg) {
    // reverse order of encoding
    for (int i = (int)msg->task.filter.size() - 1; i >= 0; --i) FindFilterOrCreate(msg->task.filter[i])->decode(msg);
  }
  Filter* FindFilterOrCreate(const FilterConfig& conf) {
    auto it = filters.find((int)conf.type);
    if (it == filters.end()) it = filters.emplace((int)conf.type, Filter::create(conf)).first;
    return it->second;
  }
  // group bookkeeping; members stay ordered by key range
  void AddGroupNode(RemoteNode* rnode) {
    PS_CHECK(rnode != nullptr);
    size_t pos = 0;
    Range<Key> kr(rnode->node.key);
    while (pos < group.size()) {
      if (kr.InLeft(Range<Key>(group[pos]->node.key))) break;
      ++pos;
    }
    group.insert(group.begin() + pos, rnode);
    keys.insert(keys.begin() + pos, kr);
  }
  void RemoveGroupNode(RemoteNode* rnode) {
    size_t n = group.size();
    PS_CHECK_EQ(n, keys.size());
    for (size_t i = 0; i < n; ++i) {
      if (group[i] == rnode) { group.erase(group.begin() + i); keys.erase(keys.begin() + i); return; }
    }
  }
  void ClearFilters() { for (auto& f : filters) delete f.second; filters.clear(); }

  Node node;
  bool alive = true;
  RequestTracker sent_req_tracker;   // requests I sent to this node
  RequestTracker recv_req_tracker;   // requests this node sent to me
  std::vector<RemoteNode*> group;    // members if this is a group node
  std::vector<Range<Key>> keys;      // members' key ranges, same order
  std::unordered_map<int, Filter*> filters;
};

}  // namespace PS
