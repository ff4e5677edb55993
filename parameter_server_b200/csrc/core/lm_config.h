// Typed application configuration of the linear methods, filled from the text
// format. Counterparts: app/linear_method/proto/linear.proto:7-101,
// learner/proto/bcd.proto:8-45, data/proto/data.proto:4-50.
#pragma once
#include "task.h"
#include "textproto.h"

namespace PS {
namespace LM {

struct LossConfig { enum Type { SQUARE = 1, LOGIT = 2, HINGE = 3, SQUARE_HINGE = 4 }; Type type = LOGIT; };
struct PenaltyConfig { enum Type { L1 = 1, L2 = 2 }; Type type = L1; std::vector<double> lambda; };
struct LearningRateConfig { enum Type { CONSTANT = 1, DECAY = 2 }; Type type = DECAY; double alpha = 1; double beta = 1; };

struct SGDConfig {
  enum Algo { STANDARD = 1, FTRL = 2 };
  Algo algo = FTRL;
  int minibatch = 1000;
  int data_buf = 1000;          // MB of prefetched minibatches
  bool ada_grad = true;
  int max_delay = 0;            // bounded delay in minibatches
  int num_data_pass = 1;
  int report_interval = 1;
  int tail_feature_freq = 0;
  double countmin_n = 1e8;
  int countmin_k = 2;
  std::vector<FilterConfig> push_filter, pull_filter;
};

struct BCDConfig {
  double feature_block_ratio = 4;
  bool random_feature_block_order = true;
  std::vector<int> prior_fea_group;
  int num_iter_for_prior_fea_group = 5;
  int max_block_delay = 0;
  int max_pass_of_data = 10;
  double epsilon = 1e-4;
  int tail_feature_freq = 0;
  int countmin_k = 2;
  double countmin_n_ratio = 2.0;
  int max_num_parallel_groups_in_preprocessing = 1000;
  int max_data_buf_size_in_mb = 1000;
  bool has_local_cache = false;
  DataConfig local_cache;
  std::vector<FilterConfig> comm_filter;
  int save_model_every_n_iter = 0;
  bool load_local_data = false;
  ParamInit init_w;            // initial weights on the servers (learner/proto/bcd.proto:40); ZERO by default
  // linear-method extensions
  double delta_init_value = 1;
  double delta_max_value = 5;
  double kkt_filter_threshold_ratio = 10;
};

struct Config {
  bool has_training_data = false, has_validation_data = false, has_model_output = false, has_model_input = false;
  DataConfig training_data, validation_data, model_output, model_input;
  LossConfig loss;
  PenaltyConfig penalty;
  LearningRateConfig learning_rate;
  bool has_async_sgd = false, has_darlin = false;
  SGDConfig async_sgd;
  BCDConfig darlin;
};

inline DataConfig ParseData(const TextNode& n) {
  DataConfig d;
  std::string f = n.str("format", "TEXT");
  d.format = f == "BIN" ? DataConfig::BIN : f == "PROTO" ? DataConfig::PROTO : DataConfig::TEXT;
  static const std::map<std::string, DataConfig::TextFormat> tf = {
      {"DENSE", DataConfig::DENSE}, {"SPARSE", DataConfig::SPARSE}, {"SPARSE_BINARY", DataConfig::SPARSE_BINARY},
      {"ADFEA", DataConfig::ADFEA}, {"LIBSVM", DataConfig::LIBSVM}, {"TERAFEA", DataConfig::TERAFEA},
      {"VW", DataConfig::VW}, {"CRITEO", DataConfig::CRITEO}};
  auto it = tf.find(n.str("text", "LIBSVM"));
  PS_CHECK(it != tf.end()) << "unknown text format " << n.str("text");
  d.text = it->second;
  d.file = n.all("file");
  d.ignore_feature_group = n.boolean("ignore_feature_group", false);
  d.max_num_files_per_worker = (int)n.integer("max_num_files_per_worker", -1);
  d.max_num_lines_per_file = (int)n.integer("max_num_lines_per_file", -1);
  d.shuffle = n.boolean("shuffle", false);
  d.replica = (int)n.integer("replica", 1);
  if (const TextNode* h = n.child("hdfs")) {
    d.has_hdfs = true;
    d.hdfs.home = h->str("home", ""); d.hdfs.ugi = h->str("ugi", ""); d.hdfs.namenode = h->str("namenode", "");
  }
  if (const TextNode* r = n.child("range")) { d.has_range = true; d.range = Range<Key>(r->integer("begin"), r->integer("end")); }
  return d;
}

inline FilterConfig ParseFilter(const TextNode& n) {
  FilterConfig f;
  std::string t = n.str("type");
  f.type = t == "KEY_CACHING" ? FilterConfig::KEY_CACHING : t == "COMPRESSING" ? FilterConfig::COMPRESSING
         : t == "FIXING_FLOAT" ? FilterConfig::FIXING_FLOAT : t == "NOISE" ? FilterConfig::NOISE
         : (FilterConfig::Type)0;
  PS_CHECK(f.type != (FilterConfig::Type)0) << "unknown filter type " << t;
  f.clear_cache_if_done = n.boolean("clear_cache_if_done", false);
  f.num_bytes = (int)n.integer("num_bytes", 3);
  f.mean = (float)n.num("mean", 0);
  f.std = (float)n.num("std", 1);
  for (auto* fp : n.children_of("fixed_point")) {
    FilterConfig::FixedFloat x;
    if (fp->has("min_value")) { x.has_min = true; x.min_value = (float)fp->num("min_value"); }
    if (fp->has("max_value")) { x.has_max = true; x.max_value = (float)fp->num("max_value"); }
    f.fixed_point.push_back(x);
  }
  return f;
}

inline Config ParseConfig(const std::string& text) {
  TextNode root = TextProtoParser::Parse(text);
  Config c;
  if (auto* n = root.child("training_data")) { c.has_training_data = true; c.training_data = ParseData(*n); }
  if (auto* n = root.child("validation_data")) { c.has_validation_data = true; c.validation_data = ParseData(*n); }
  if (auto* n = root.child("model_output")) { c.has_model_output = true; c.model_output = ParseData(*n); }
  if (auto* n = root.child("model_input")) { c.has_model_input = true; c.model_input = ParseData(*n); }
  if (auto* n = root.child("loss")) {
    std::string t = n->str("type", "LOGIT");
    c.loss.type = t == "SQUARE" ? LossConfig::SQUARE : t == "HINGE" ? LossConfig::HINGE
                : t == "SQUARE_HINGE" ? LossConfig::SQUARE_HINGE : LossConfig::LOGIT;
  }
  if (auto* n = root.child("penalty")) {
    c.penalty.type = n->str("type", "L1") == "L2" ? PenaltyConfig::L2 : PenaltyConfig::L1;
    for (auto& v : n->all("lambda")) c.penalty.lambda.push_back(atof(v.c_str()));
  }
  if (auto* n = root.child("learning_rate")) {
    c.learning_rate.type = n->str("type", "DECAY") == "CONSTANT" ? LearningRateConfig::CONSTANT : LearningRateConfig::DECAY;
    c.learning_rate.alpha = n->num("alpha", 1);
    c.learning_rate.beta = n->num("beta", 1);
  }
  if (auto* n = root.child("async_sgd")) {
    c.has_async_sgd = true;
    SGDConfig& s = c.async_sgd;
    s.algo = n->str("algo", "FTRL") == "STANDARD" ? SGDConfig::STANDARD : SGDConfig::FTRL;
    s.minibatch = (int)n->integer("minibatch", 1000);
    s.data_buf = (int)n->integer("data_buf", 1000);
    s.ada_grad = n->boolean("ada_grad", true);
    s.max_delay = (int)n->integer("max_delay", 0);
    s.num_data_pass = (int)n->integer("num_data_pass", 1);
    s.report_interval = (int)n->integer("report_interval", 1);
    s.tail_feature_freq = (int)n->integer("tail_feature_freq", 0);
    s.countmin_n = n->num("countmin_n", 1e8);
    s.countmin_k = (int)n->integer("countmin_k", 2);
    for (auto* f : n->children_of("push_filter")) s.push_filter.push_back(ParseFilter(*f));
    for (auto* f : n->children_of("pull_filter")) s.pull_filter.push_back(ParseFilter(*f));
  }
  if (auto* n = root.child("darlin")) {
    c.has_darlin = true;
    BCDConfig& b = c.darlin;
    b.feature_block_ratio = n->num("feature_block_ratio", 4);
    b.random_feature_block_order = n->boolean("random_feature_block_order", true);
    for (auto& v : n->all("prior_fea_group")) b.prior_fea_group.push_back(atoi(v.c_str()));
    b.num_iter_for_prior_fea_group = (int)n->integer("num_iter_for_prior_fea_group", 5);
    b.max_block_delay = (int)n->integer("max_block_delay", 0);
    b.max_pass_of_data = (int)n->integer("max_pass_of_data", 10);
    b.epsilon = n->num("epsilon", 1e-4);
    b.tail_feature_freq = (int)n->integer("tail_feature_freq", 0);
    b.countmin_k = (int)n->integer("countmin_k", 2);
    b.countmin_n_ratio = n->num("countmin_n_ratio", 2.0);
    b.max_num_parallel_groups_in_preprocessing = (int)n->integer("max_num_parallel_groups_in_preprocessing", 1000);
    b.max_data_buf_size_in_mb = (int)n->integer("max_data_buf_size_in_mb", 1000);
    if (auto* lc = n->child("local_cache")) { b.has_local_cache = true; b.local_cache = ParseData(*lc); }
    for (auto* f : n->children_of("comm_filter")) b.comm_filter.push_back(ParseFilter(*f));
    b.save_model_every_n_iter = (int)n->integer("save_model_every_n_iter", 0);
    b.load_local_data = n->boolean("load_local_data", false);
    if (const TextNode* w = n->child("init_w")) {
      static const std::map<std::string, ParamInit::Type> types = {
          {"ZERO", ParamInit::ZERO}, {"CONSTANT", ParamInit::CONSTANT}, {"GAUSSIAN", ParamInit::GAUSSIAN},
          {"FILE", ParamInit::FILE}, {"CLONE", ParamInit::CLONE}};
      auto it = types.find(w->str("type", "ZERO"));
      PS_CHECK(it != types.end()) << "unknown init_w type " << w->str("type");
      b.init_w.type = it->second;
      b.init_w.constant = w->num("constant", 1);
      b.init_w.mean = w->num("mean", 0);
      b.init_w.std = w->num("std", 1);
      b.init_w.file_name = w->str("file_name", "");
    }
    b.delta_init_value = n->num("delta_init_value", 1);
    b.delta_max_value = n->num("delta_max_value", 5);
    b.kkt_filter_threshold_ratio = n->num("kkt_filter_threshold_ratio", 10);
  }
  return c;
}

}  // namespace LM
}  // namespace PS
