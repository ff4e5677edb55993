// Shared parameters: the Push/Pull protocol on top of Customer, and the three
// containers KVVector (sorted key/value arrays per channel, optional
// per-timestamp aggregation buffers), KVMap (hash map whose entry type runs the
// optimiser inside SetValue) and KVLayer (dense tensors keyed by layer id).
// Counterparts: parameter/parameter.h:7-77, parameter/parameter.cc:5-49,
// parameter/kv_vector.h:31-262, parameter/kv_map.h:9-130,
// parameter/kv_layer.h:10-210, parameter/kv_store.h:1-7.
#pragma once
#include <fstream>
#include "customer.h"
#include "ordered_match.h"
#include "postoffice.h"

namespace PS {

class Parameter : public Customer {
 public:
  explicit Parameter(int id, Postoffice* po = nullptr) : Customer(id, po) {}
  virtual ~Parameter() {}
  typedef std::initializer_list<int> Timestamps;
  typedef std::initializer_list<FilterConfig> Filters;

  // Builds the header of a push or pull: key channel, explicit timestamp,
  // timestamps to wait for at the receiver, filters, key range.
  static Task Request(int channel, int ts = Message::kInvalidTime, const std::vector<int>& wait = {},
                      const std::vector<FilterConfig>& filters = {}, const Range<Key>& key_range = Range<Key>::All()) {
    Task req;
    req.request = true;
    req.key_channel = channel;
    if (ts > Message::kInvalidTime) req.set_time(ts);
    for (int t : wait) if (t > Message::kInvalidTime) req.wait_time.push_back(t);
    for (const auto& f : filters) req.filter.push_back(f);
    req.set_key_range(key_range);
    return req;
  }
  int Push(Message* msg) { msg->task.mutable_param()->push = true; return Submit(msg); }
  int Pull(Message* msg) { msg->task.mutable_param()->push = false; return Submit(msg); }

  virtual void WriteToFile(const std::string& file) {}

  void ProcessRequest(Message* request) override {
    const ParamCall& call = request->task.param;
    bool push = call.push;
    if (push) {
      SetValue(request);
      if (call.replica) SetReplica(request);
    } else {
      // the response carries the request's header (channel, key range, filters) and keys
      Message response;
      response.task = request->task;
      response.task.wait_time.clear();
      response.key = request->key;
      response.task.has_key = request->has_key();
      if (call.replica) GetReplica(&response); else GetValue(&response);
      Reply(request, &response);
    }
  }
  void ProcessResponse(Message* response) override {
    const ParamCall& call = response->task.param;
    if (!call.push) {
      if (call.replica) Recover(response); else SetValue(response);
    }
  }

 protected:
  // fill `msg` with my values for msg->key
  virtual void GetValue(Message* msg) = 0;
  // merge the values of `msg` into mine
  virtual void SetValue(const Message* msg) = 0;
  // replication hooks
  virtual void GetReplica(Message* msg) {}
  virtual void SetReplica(const Message* msg) {}
  virtual void Recover(Message* msg) {}
};

// ================================================================= KVVector
template <typename K, typename V>
class KVVector : public Parameter {
 public:
  // buffer_value: received values are kept in per-timestamp buffers (summed
  // over senders) instead of being merged into the channel's value array.
  // k: values per key.
  KVVector(bool buffer_value = false, int k = 1, int id = -1, Postoffice* po = nullptr)
      : Parameter(id >= 0 ? id : (po ? po : &Postoffice::instance())->manager().NextCustomerID(), po),
        k_(k), buffer_value_(buffer_value) {
    PS_CHECK_GT(k, 0);
  }
  virtual ~KVVector() {}
  using Parameter::Push;
  using Parameter::Pull;

  struct KVPairs {
    SArray<K> key;    // sorted, unique
    SArray<V> value;  // size = key.size() * k
  };
  struct Buffer {
    int channel = 0;
    SizeR idx_range;                 // positions in the channel's key list
    std::vector<SArray<V>> values;   // one array per pushed value array
  };
  KVPairs& operator[](int chl) { Lock l(mu_); return data_[chl]; }
  void Clear(int chl) { Lock l(mu_); data_.erase(chl); }
  Buffer& buffer(int ts) { Lock l(mu_); return buffer_[ts]; }
  void ClearBuffer(int ts) { Lock l(mu_); buffer_.erase(ts); }
  void ClearFilter() { Lock l(mu_); key_filter_.clear(); }
  int k() const { return k_; }

  // Push (key, value...) to the server group; returns the timestamp.
  int Push(const Task& request, const SArray<K>& keys, const std::vector<SArray<V>>& values = {},
           const std::function<void()>& callback = nullptr) {
    Message push(request);
    push.recver = kServerGroup;
    push.set_key(keys);
    for (const auto& v : values) { if (!v.empty()) PS_CHECK_EQ(v.size(), keys.size() * k_); push.add_value(v); }
    if (callback) push.callback = callback;
    return Parameter::Push(&push);
  }
  // Pull the values of `keys` from the server group into channel request.key_channel
  // (or into buffer(timestamp) with buffer_value).
  int Pull(const Task& request, const SArray<K>& keys, const std::function<void()>& callback = nullptr) {
    Message pull(request);
    pull.recver = kServerGroup;
    pull.set_key(keys);
    if (callback) pull.callback = callback;
    return Parameter::Pull(&pull);
  }
  void Slice(const Message& request, const std::vector<Range<Key>>& krs, std::vector<Message*>* msgs) override {
    for (auto m : *msgs) { m->task = request.task; }
    SliceKOFVMessage<K>(request, krs, msgs);
  }

  void WriteToFile(const std::string& file) override {
    Lock l(mu_);
    std::ofstream out(file);
    for (auto& ch : data_) {
      auto& kv = ch.second;
      for (size_t i = 0; i < kv.key.size(); ++i) {
        if (kv.value.size() <= i * k_) break;
        bool nz = false;
        for (int j = 0; j < k_; ++j) { V v = kv.value[i * k_ + j]; nz |= (v != 0 && v == v); }
        if (!nz) continue;
        out << kv.key[i];
        for (int j = 0; j < k_; ++j) out << "\t" << kv.value[i * k_ + j];
        out << "\n";
      }
    }
  }

 protected:
  void GetValue(Message* msg) override {
    SArray<K> recv_key(msg->key);
    Lock l(mu_);
    int chl = msg->task.key_channel;
    if (msg->task.has_param && msg->task.param.has_tail_filter && msg->task.param.tail_filter.has_freq_threshold) {
      // reply with the keys whose estimated frequency passes the threshold
      auto& filter = key_filter_[chl];
      msg->clear_value();
      msg->set_key(filter.QueryKeys(recv_key, msg->task.param.tail_filter.freq_threshold));
      return;
    }
    auto& kv = data_[chl];
    msg->clear_value();
    if (recv_key.empty()) return;
    // ordered match of my (key, value) onto the requested keys
    SArray<V> val;
    if (kv.value.size() != kv.key.size() * k_) { kv.value.resize(kv.key.size() * k_); }
    size_t n = ParallelOrderedMatch(kv.key, kv.value, recv_key, &val, k_, AssignOp::ASSIGN);
    (void)n;
    msg->add_value(val);
  }

  void SetValue(const Message* msg) override {
    SArray<K> recv_key(msg->key);
    int chl = msg->task.key_channel;
    Lock l(mu_);
    if (msg->task.has_param && msg->task.param.has_tail_filter && msg->task.param.tail_filter.insert_count) {
      // (key, count) pairs feed the channel's count-min sketch
      PS_CHECK_EQ(msg->value.size(), (size_t)1);
      SArray<uint8_t> cnt(msg->value[0]);
      auto& filter = key_filter_[chl];
      if (filter.Empty()) {
        const auto& tf = msg->task.param.tail_filter;
        filter.Resize(std::max(tf.countmin_n, 64), std::max(tf.countmin_k, 1));
      }
      filter.InsertKeys(recv_key, cnt);
      return;
    }
    auto& kv = data_[chl];
    if (msg->value.empty()) {
      // keys only: merge them into my key set, values are reset
      if (recv_key.empty()) return;
      kv.key = kv.key.SetUnion(recv_key);
      kv.value.clear();
      return;
    }
    if (recv_key.empty()) return;
    if (!buffer_value_) {
      for (size_t i = 0; i < msg->value.size() && i < 1; ++i) {
        SArray<V> recv_val(msg->value[i]);
        if (kv.key.empty()) { kv.key = recv_key.Clone(); }
        AssignOp op = msg->task.request ? AssignOp::PLUS : AssignOp::ASSIGN;
        if (msg->task.has_param && msg->task.param.op != 0) op = (AssignOp)msg->task.param.op;
        ParallelOrderedMatch(recv_key, recv_val, kv.key, &kv.value, k_, op);
      }
      return;
    }
    // aggregate into the buffer of this timestamp, over the positions of my key
    // list that the message's key range covers; senders are summed
    int ts = msg->task.time;
    auto& buf = buffer_[ts];
    Range<Key> kr = msg->task.has_key_range ? msg->task.key_range : Range<Key>::All();
    SizeR idx = kv.key.FindRange(kr);
    if (buf.values.empty()) {
      buf.values.resize(msg->value.size());
      buf.idx_range = idx;
      buf.channel = chl;
    } else {
      PS_CHECK(buf.idx_range == idx) << "timestamp " << ts << " reused for another key range";
      PS_CHECK_EQ(buf.channel, chl);
      if (buf.values.size() < msg->value.size()) buf.values.resize(msg->value.size());
    }
    SArray<K> my_key = kv.key.Segment(buf.idx_range);
    for (size_t i = 0; i < msg->value.size(); ++i) {
      SArray<V> recv_val(msg->value[i]);
      if (recv_val.empty()) continue;
      int k = (int)(recv_val.size() / recv_key.size());  // not necessarily k_
      auto& dst = buf.values[i];
      if (dst.size() != my_key.size() * k) { dst.resize(my_key.size() * k); dst.SetZero(); }
      ParallelOrderedMatch(recv_key, recv_val, my_key, &dst, k, AssignOp::PLUS);
    }
  }

  int k_;
  bool buffer_value_;
  std::unordered_map<int, KVPairs> data_;
  std::unordered_map<int, Buffer> buffer_;
  std::unordered_map<int, FreqencyFilter<K, uint8_t>> key_filter_;
  std::mutex mu_;
};

// ================================================================= KVMap
// E must provide   void Get(V* data, void* state);  void Set(const V* data, void* state);
// S must provide   void Update();      (called once per push message)
template <typename K, typename V, typename E, typename S>
class KVMap : public Parameter {
 public:
  KVMap(int k = 1, int id = -1, Postoffice* po = nullptr)
      : Parameter(id >= 0 ? id : (po ? po : &Postoffice::instance())->manager().NextCustomerID(), po), k_(k) {
    PS_CHECK_GT(k, 0);
  }
  virtual ~KVMap() {}
  void set_state(const S& s) { state_ = s; }
  S& state() { return state_; }
  size_t size() { Lock l(mu_); return data_.size(); }

  void Slice(const Message& request, const std::vector<Range<Key>>& krs, std::vector<Message*>* msgs) override {
    for (auto m : *msgs) { m->task = request.task; }
    SliceKOFVMessage<K>(request, krs, msgs);
  }
  // one line per stored key with a non-zero value: key <TAB> value
  void WriteToFile(const std::string& file) override {
    Lock l(mu_);
    std::ofstream out(file);
    PS_CHECK(out.good()) << "cannot write " << file;
    V v;
    for (auto& e : data_) {
      e.second.Get(&v, &state_);
      if (v != 0) out << e.first << "\t" << v << "\n";
    }
  }

 protected:
  void GetValue(Message* msg) override {
    SArray<K> key(msg->key);
    size_t n = key.size();
    SArray<V> val(n * k_);
    Lock l(mu_);
    for (size_t i = 0; i < n; ++i) data_[key[i]].Get(val.data() + i * k_, &state_);
    msg->clear_value();
    msg->add_value(val);
  }
  void SetValue(const Message* msg) override {
    SArray<K> key(msg->key);
    size_t n = key.size();
    if (msg->value.empty()) return;
    PS_CHECK_EQ(msg->value.size(), (size_t)1);
    SArray<V> val(msg->value[0]);
    PS_CHECK_EQ(n * k_, val.size());
    Lock l(mu_);
    for (size_t i = 0; i < n; ++i) data_[key[i]].Set(val.data() + i * k_, &state_);
    state_.Update();
  }
  int k_;
  S state_;
  std::unordered_map<K, E> data_;
  std::mutex mu_;
};

// ================================================================= KVLayer
// Updater must provide  void Init(int id, size_t n, V* data);
//                       void Update(int id, size_t n, const V* recv, V* data);
template <typename V, class Updater>
class KVLayer : public Parameter {
 public:
  // layers with fewer than partition_thr elements live on one server; larger ones are
  // split evenly over all servers
  KVLayer(size_t partition_thr = 1000, int id = -1, Postoffice* po = nullptr)
      : Parameter(id >= 0 ? id : (po ? po : &Postoffice::instance())->manager().NextCustomerID(), po),
        partition_thr_(partition_thr) {}
  virtual ~KVLayer() {}
  void set_updater(Updater* u) { updater_ = u; }
  SArray<V> operator[](int key) { Lock l(mu_); return layer_[key]; }
  SArray<V> layer(int key) { Lock l(mu_); return layer_[key]; }

  // Push `data` (layer id = task.key_channel); zero_copy: the caller keeps `data` alive until acked
  int Push(const Task& task, V* data, size_t size, bool zero_copy = false) {
    SArray<V> val;
    if (zero_copy) val = SArray<V>::Wrap(data, size); else val.CopyFrom(data, size);
    Message push(task);
    push.recver = kServerGroup;
    push.add_value(val);
    return Parameter::Push(&push);
  }
  // Pull layer task.key_channel into `data`
  int Pull(const Task& task, V* data, size_t size, const std::function<void()>& callback = nullptr) {
    int id = task.key_channel;
    { Lock l(mu_); layer_[id] = SArray<V>::Wrap(data, size); }
    Message pull(task);
    pull.recver = kServerGroup;
    // the value array only announces the size; the servers send their segments back
    SArray<V> announce = SArray<V>::Wrap(data, size);
    pull.add_value(announce);
    if (callback) pull.callback = callback;
    return Parameter::Pull(&pull);
  }

  void Slice(const Message& request, const std::vector<Range<Key>>& krs, std::vector<Message*>* msgs) override {
    size_t n = krs.size();
    int id = request.task.key_channel;
    PS_CHECK_EQ(request.value.size(), (size_t)1);
    SArray<V> val(request.value[0]);
    const bool pull = request.task.has_param && !request.task.param.push;
    for (size_t i = 0; i < n; ++i) {
      Message* m = (*msgs)[i];
      NodeID recver = m->recver;
      m->task = request.task;
      m->recver = recver;
      m->valid = true;
      m->clear_data();
      SizeR seg;
      if (val.size() < partition_thr_) {
        // the whole layer goes to one server picked by its id
        if ((size_t)((id * 991) % n) != i) { m->valid = false; continue; }
        seg = SizeR(0, val.size());
      } else {
        seg = SizeR(0, val.size()).EvenDivide(n, i);
      }
      // the element range travels in key_range
      m->task.set_key_range(Range<Key>(seg.begin(), seg.end()));
      if (pull) {
        SArray<V> none;
        m->add_value(none);
        m->task.msg = std::to_string(val.size());
      } else {
        m->add_value(val.Segment(seg));
        m->task.msg = std::to_string(val.size());
      }
    }
  }
  void WriteToFile(const std::string& file) override {
    Lock l(mu_);
    std::ofstream out(file);
    for (auto& kv : layer_) for (size_t i = 0; i < kv.second.size(); ++i)
      if (kv.second[i] != 0) out << kv.first << ":" << i << "\t" << kv.second[i] << "\n";
  }

 protected:
  void GetValue(Message* msg) override {
    // server: return my segment of the layer
    int id = msg->task.key_channel;
    Lock l(mu_);
    Range<Key> kr = msg->task.key_range;
    auto& mine = layer_[id];
    msg->clear_value();
    SArray<V> seg;
    if (mine.size() >= kr.size()) seg = mine.Segment(SizeR(0, kr.size()));
    else { seg.resize(kr.size()); seg.SetZero(); }
    msg->add_value(seg);
  }
  void SetValue(const Message* msg) override {
    int id = msg->task.key_channel;
    if (msg->value.empty()) return;
    SArray<V> recv(msg->value[0]);
    Range<Key> kr = msg->task.key_range;
    Lock l(mu_);
    if (msg->task.request) {
      // server side of a push: my part of layer `id` is the received segment's size
      auto& mine = layer_[id];
      if (mine.size() != recv.size()) {
        mine.resize(recv.size());
        mine.SetZero();
        if (updater_) updater_->Init(id, mine.size(), mine.data());
      }
      if (updater_) updater_->Update(id, recv.size(), recv.data(), mine.data());
      else for (size_t i = 0; i < recv.size(); ++i) mine[i] += recv[i];
    } else {
      // worker side of a pull: copy the segment into place
      auto& mine = layer_[id];
      PS_CHECK_LE(kr.end(), mine.size());
      PS_CHECK_EQ(kr.size(), recv.size());
      if (recv.size()) memcpy(mine.data() + kr.begin(), recv.data(), recv.size() * sizeof(V));
    }
  }
  size_t partition_thr_;
  Updater* updater_ = nullptr;
  std::unordered_map<int, SArray<V>> layer_;
  std::mutex mu_;
};

// Placeholder for a generic disk/remote backed store (the reference only
// declares it: parameter/kv_store.h:1-7).
class KVStore {};

}  // namespace PS
