// Message = Task header + optional key array + value arrays (zero-copy byte
// views) + local delivery flags; and the key-range slicer used by every
// key/value Push and Pull. Counterpart of system/message.h:10-147.
#pragma once
#include "sarray.h"
#include "task.h"

namespace PS {

struct Message;
typedef std::shared_ptr<Message> MessagePtr;

struct Message {
  static const int kInvalidTime = -1;
  Message() {}
  explicit Message(const Task& tk) : task(tk) {}
  Message(const NodeID& dest, int time = kInvalidTime, int wait_time = kInvalidTime) : recver(dest) {
    if (time != kInvalidTime) task.set_time(time);
    if (wait_time != kInvalidTime) task.wait_time.push_back(wait_time);
  }
  Task task;
  SArray<char> key;
  std::vector<SArray<char>> value;

  // not sent over the wire
  NodeID sender, recver;
  bool replied = false;    // a reply has been sent for this request
  bool finished = true;    // set false in ProcessRequest to defer completion
  bool valid = true;       // false: do not send (no key-range overlap)
  bool terminate = false;  // stops the I/O threads
  std::function<void()> callback;  // runs when every recipient has answered

  bool has_key() const { return !key.empty(); }
  void clear_key() { task.has_key = false; key.clear(); }
  void clear_value() { task.value_type.clear(); value.clear(); }
  void clear_data() { clear_key(); clear_value(); }
  template <typename K>
  void set_key(const SArray<K>& k) {
    task.key_type = EncodeType<K>();
    task.has_key = true;
    key = SArray<char>(k);
    if (!task.has_key_range) task.set_key_range(Range<Key>::All());
  }
  template <typename V>
  void add_value(const SArray<V>& v) {
    task.value_type.push_back(EncodeType<V>());
    value.push_back(SArray<char>(v));
  }
  size_t mem_size() const {
    size_t n = task.Serialize().size() + key.size();
    for (const auto& v : value) n += v.size();
    return n;
  }
  std::string ShortDebugString() const {
    std::ostringstream ss;
    ss << sender << "=>" << recver << " " << task.ShortDebugString() << " key[" << key.size() << "]";
    for (const auto& v : value) ss << " val[" << v.size() << "]";
    return ss.str();
  }
};

// Splits a message whose keys are sorted into one message per key range
// (zero-copy segments). A range that does not intersect the message's own
// key_range gives valid=false; an intersecting range with no keys still gives a
// valid, empty message so that the receiver can count it.
template <typename K>
void SliceKOFVMessage(const Message& msg, const std::vector<Range<Key>>& krs, std::vector<Message*>* rets) {
  PS_CHECK_EQ(rets->size(), krs.size());
  size_t n = krs.size();
  std::vector<size_t> pos(n + 1, 0);
  SArray<K> key(msg.key);
  Range<Key> msg_range = msg.task.has_key_range ? msg.task.key_range : Range<Key>::All();
  for (size_t i = 0; i < n; ++i) {
    // boundaries are clamped into the message's own key range
    if (i == 0) pos[0] = std::lower_bound(key.begin(), key.end(), (K)msg_range.Project(krs[0].begin())) - key.begin();
    else PS_CHECK_EQ(krs[i - 1].end(), krs[i].begin());
    pos[i + 1] = std::lower_bound(key.begin(), key.end(), (K)msg_range.Project(krs[i].end())) - key.begin();
  }
  for (size_t i = 0; i < n; ++i) {
    Message* ret = (*rets)[i];
    if (krs[i].SetIntersection(msg_range).empty()) { ret->valid = false; continue; }
    ret->valid = true;  // an empty slice of an owned range is still sent
    if (key.empty()) continue;
    SizeR lr(pos[i], pos[i + 1]);
    ret->set_key(key.Segment(lr));
    ret->value.clear();
    ret->task.value_type = msg.task.value_type;
    for (const auto& v : msg.value) {
      size_t k = v.size() / key.size();  // bytes per key
      PS_CHECK_EQ(key.size() * k, v.size());
      ret->value.push_back(v.Segment(SizeR(lr.begin() * k, lr.end() * k)));
    }
  }
}

}  // namespace PS
