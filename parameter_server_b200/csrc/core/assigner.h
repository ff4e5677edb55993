// NodeAssigner: ranks and key ranges for joining nodes. DataAssigner: splits a
// file list over workers. Counterpart of system/assigner.h:9-57, assigner.cc:5-38.
#pragma once
#include <algorithm>
#include <random>
#include <string>
#include <vector>
#include "task.h"

namespace PS {

class NodeAssigner {
 public:
  NodeAssigner(int num_servers, Range<Key> key_range) : num_servers_(num_servers), key_range_(key_range) {}
  // servers: the rank-th even slice of the key range; workers: the whole range. A node whose id is
  // its role letter plus a number ("S3", "W0", the ids the launch scripts give) gets that number as
  // its rank when it is free, so that ranks do not depend on the order in which nodes register;
  // any other id takes the lowest free rank.
  void assign(Node* node) {
    Range<Key> kr = key_range_;
    int rank = 0;
    if (node->role == Node::SERVER) {
      rank = pick(node->id, 'S', num_servers_, &server_taken_);
      PS_CHECK_LT(rank, num_servers_) << "more servers than -num_servers";
      kr = key_range_.EvenDivide(num_servers_, rank);
    } else if (node->role == Node::WORKER) {
      rank = pick(node->id, 'W', 1 << 30, &worker_taken_);
    }
    node->rank = rank;
    node->key = kr;
  }
  void remove(const Node& node) {}  // ranges of the remaining servers are not re-balanced
 private:
  static int pick(const std::string& id, char letter, int limit, std::vector<bool>* taken) {
    int want = -1;
    if (id.size() > 1 && id.size() < 9 && id[0] == letter &&
        std::all_of(id.begin() + 1, id.end(), [](char c) { return c >= '0' && c <= '9'; }))
      want = std::atoi(id.c_str() + 1);
    auto is_free = [taken](int r) { return r >= (int)taken->size() || !(*taken)[r]; };
    int rank = (want >= 0 && want < limit && is_free(want)) ? want : 0;
    if (rank != want) while (!is_free(rank)) ++rank;
    if (rank >= (int)taken->size()) taken->resize(rank + 1, false);
    (*taken)[rank] = true;
    return rank;
  }
  int num_servers_ = 0;
  std::vector<bool> server_taken_, worker_taken_;
  Range<Key> key_range_;
};

class DataAssigner {
 public:
  DataAssigner() {}
  DataAssigner(const DataConfig& data, int num, bool local) { set(data, num, local); }
  // `num` parts; with `local` every worker reads the same config
  void set(const DataConfig& data, int num, bool local) {
    parts_.clear();
    cur_ = 0;
    if (local) {
      for (int i = 0; i < num; ++i) parts_.push_back(data);
      return;
    }
    std::vector<std::string> files = data.file;
    if (data.shuffle) { std::mt19937 g(7); std::shuffle(files.begin(), files.end(), g); }
    int replica = std::max(1, data.replica);
    for (int r = 0; r < replica; ++r) {
      for (int i = 0; i < num; ++i) {
        DataConfig part = data;
        part.file.clear();
        for (size_t f = i; f < files.size(); f += num) {
          if (data.max_num_files_per_worker >= 0 && (int)part.file.size() >= data.max_num_files_per_worker) break;
          part.file.push_back(files[f]);
        }
        parts_.push_back(part);
      }
    }
  }
  bool next(DataConfig* data) {
    if (cur_ >= parts_.size()) return false;
    *data = parts_[cur_++];
    return true;
  }
  size_t size() const { return parts_.size(); }
 private:
  std::vector<DataConfig> parts_;
  size_t cur_ = 0;
};

}  // namespace PS
