// Environment manager: collects variables the plugin wants NCCL to see (NCCL_* defaults chosen
// by the platform) and publishes them by building a fresh `environ` array and swapping the
// pointer, never calling setenv() — other threads may be walking the old array, which is left
// intact and never freed (reference: include/nccl_ofi_environ.h:18-151).
#pragma once
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace b200net {

class EnvManager {
 public:
  static EnvManager& instance();
  // Record name=value. overwrite=false keeps a value already present in the process environment.
  void insert_envvar(const std::string& name, const std::string& value, bool overwrite);
  // Build the new array (old entries + recorded ones) and store it into *environ_ptr.
  void update_environment(char*** environ_ptr);
  size_t pending() const;
  void clear_for_testing();

 private:
  struct Entry { std::string value; bool overwrite; };
  mutable std::mutex mu_;
  std::map<std::string, Entry> vars_;
  std::vector<char**> retired_;  // arrays that were once published: kept alive forever
};

}  // namespace b200net
