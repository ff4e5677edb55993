// Node options ("flags") and environment bootstrap.
// Flag names follow the reference: -num_servers -num_workers -num_threads
// -num_replicas -my_node -scheduler -interface (system/env.cc:10-18),
// -app_file -app_conf -key_start -key_end (system/manager.cc:11-15),
// -bind_to -local (system/van.cc:10-11), -report_interval
// (system/postoffice.cc:8-11), -log_dir. When -my_node is absent the role and
// addresses come from DMLC_* or MPI rank variables (system/env.cc:45-93).
#pragma once
#include "common.h"
#include "task.h"

namespace PS {

struct Options {
  int num_servers = 0;
  int num_workers = 0;
  int num_threads = 2;
  int num_replicas = 0;
  std::string my_node = "role:SCHEDULER,hostname:'127.0.0.1',port:8000,id:'H'";
  std::string scheduler = "role:SCHEDULER,hostname:'127.0.0.1',port:8000,id:'H'";
  std::string interface;
  std::string app_file;
  std::string app_conf;
  uint64_t key_start = 0;
  uint64_t key_end = kMaxKey;
  int bind_to = 0;
  bool local = false;         // unix-domain sockets instead of tcp
  int report_interval = 0;    // seconds between heartbeat reports, 0 = off
  std::string log_dir;
  bool exit_on_scheduler_loss = true;
  // process-wide settings of the readers (data/stream_reader.h:104, data/text_parser.cc:163,
  // util/filelinereader.cc:29 in the reference, where they are global flags too)
  uint64_t hash_kernel = 0;   // >0: every feature id is taken modulo this
  bool shuffle_fea_id = false;  // TERAFEA ids are mixed by a hash
  int line_limit = 0;         // >0: at most this many lines are read from a text file
  std::vector<std::string> rest;  // unparsed arguments

  // "-name value", "-name=value", "--name value"; bool flags may omit the value
  static Options Parse(const std::vector<std::string>& args);
  static Options Parse(int argc, char** argv) {
    std::vector<std::string> a;
    for (int i = 1; i < argc; ++i) a.push_back(argv[i]);
    return Parse(a);
  }
  // fills my_node/scheduler/num_* from DMLC_PS_ROOT_URI, DMLC_PS_ROOT_PORT,
  // DMLC_NUM_WORKER, DMLC_NUM_SERVER, DMLC_ROLE, or PMI_RANK / OMPI_COMM_WORLD_RANK
  void InitFromEnv();
};

class Env {
 public:
  // picks a free tcp port on this machine
  static int FreePort();
  // first non-loopback IPv4 address (or of `interface`), "127.0.0.1" if none
  static std::string LocalIP(const std::string& interface = "");
};

}  // namespace PS
