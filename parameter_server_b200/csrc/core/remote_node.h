// Per-peer state held by an Executor: liveness, which timestamps have been
// sent/received and finished, group membership ordered by key range, and the
// peer's own filter instances (so key-cache state is per peer).
// Counterpart of system/remote_node.h:13-65, system/remote_node.cc:7-56.
#pragma once
#include <memory>
#include "filter.h"

namespace PS {

// Which integer timestamps are finished: a bit set in 64-bit words that grows on demand. A timestamp
// that was never started counts as unfinished; negative ones (no dependency) as finished.
class RequestTracker {
 public:
  static constexpr int kMaxTimestamp = 100000000;
  void Start(int ts) { Word(ts) &= ~Bit(ts); }
  void Finish(int ts) { Word(ts) |= Bit(ts); }
  bool IsFinished(int ts) const {
    if (ts < 0) return true;
    const size_t w = (size_t)ts >> 6;
    return w < words_.size() && (words_[w] & Bit(ts)) != 0;
  }
 private:
  static uint64_t Bit(int ts) { return 1ull << (ts & 63); }
  uint64_t& Word(int ts) {
    PS_CHECK_GE(ts, 0);
    PS_CHECK_LT(ts, kMaxTimestamp);
    const size_t w = (size_t)ts >> 6;
    if (w >= words_.size()) words_.resize(w + w / 2 + 4, 0);
    return words_[w];
  }
  std::vector<uint64_t> words_;
};

struct RemoteNode {
  // a message passes the filters named in its header in order when it leaves, in reverse when it arrives
  void EncodeMessage(Message* msg) {
    for (const FilterConfig& conf : msg->task.filter) FilterFor(conf)->encode(msg);
  }
  void DecodeMessage(Message* msg) {
    const auto& chain = msg->task.filter;
    for (auto it = chain.rbegin(); it != chain.rend(); ++it) FilterFor(*it)->decode(msg);
  }
  // this peer's instance of a filter type, made on first use
  Filter* FilterFor(const FilterConfig& conf) {
    std::unique_ptr<Filter>& f = filters[(int)conf.type];
    if (!f) f.reset(Filter::create(conf));
    return f.get();
  }
  void ClearFilters() { filters.clear(); }

  // Group bookkeeping (this entry stands for a group id): members and their key ranges, kept in key
  // order so that a sliced message lines up with the members.
  void AddGroupNode(RemoteNode* member) {
    PS_CHECK(member != nullptr);
    const Range<Key> kr(member->node.key);
    size_t at = 0;
    while (at < group.size() && !kr.InLeft(Range<Key>(group[at]->node.key))) ++at;
    group.insert(group.begin() + at, member);
    keys.insert(keys.begin() + at, kr);
  }
  void RemoveGroupNode(RemoteNode* member) {
    PS_CHECK_EQ(group.size(), keys.size());
    auto it = std::find(group.begin(), group.end(), member);
    if (it == group.end()) return;
    keys.erase(keys.begin() + (it - group.begin()));
    group.erase(it);
  }

  Node node;
  bool alive = true;
  RequestTracker sent_req_tracker;   // requests I sent to this node
  RequestTracker recv_req_tracker;   // requests this node sent to me
  std::vector<RemoteNode*> group;    // members if this is a group node
  std::vector<Range<Key>> keys;      // members' key ranges, same order
  std::unordered_map<int, std::unique_ptr<Filter>> filters;
};

}  // namespace PS
