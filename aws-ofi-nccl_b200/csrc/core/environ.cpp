#include "b200net/environ.h"

#include <cstdlib>
#include <cstring>

namespace b200net {

EnvManager& EnvManager::instance() {
  static EnvManager* m = new EnvManager();
  return *m;
}

void EnvManager::insert_envvar(const std::string& name, const std::string& value, bool overwrite) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = vars_.find(name);
  if (it != vars_.end() && !overwrite) return;  // first writer wins unless told otherwise
  vars_[name] = Entry{value, overwrite};
}

size_t EnvManager::pending() const {
  std::lock_guard<std::mutex> g(mu_);
  return vars_.size();
}

void EnvManager::clear_for_testing() {
  std::lock_guard<std::mutex> g(mu_);
  vars_.clear();
}

void EnvManager::update_environment(char*** environ_ptr) {
  std::lock_guard<std::mutex> g(mu_);
  if (vars_.empty()) return;
  char** old = *environ_ptr;
  std::vector<char*> out;
  std::map<std::string, bool> handled;
  for (char** e = old; e && *e; ++e) {
    const char* eq = strchr(*e, '=');
    const std::string key = eq ? std::string(*e, eq - *e) : std::string(*e);
    auto it = vars_.find(key);
    if (it != vars_.end()) {
      handled[key] = true;
      if (it->second.overwrite) {
        out.push_back(strdup((key + "=" + it->second.value).c_str()));
        continue;
      }
    }
    out.push_back(*e);  // strings of the old array are shared, never freed
  }
  for (auto& [key, ent] : vars_) {
    if (!handled.count(key)) out.push_back(strdup((key + "=" + ent.value).c_str()));
  }
  char** fresh = static_cast<char**>(malloc(sizeof(char*) * (out.size() + 1)));
  memcpy(fresh, out.data(), sizeof(char*) * out.size());
  fresh[out.size()] = nullptr;
  // publish with one pointer store; readers of the old array keep a consistent view
  __atomic_store_n(environ_ptr, fresh, __ATOMIC_RELEASE);
  retired_.push_back(old);
  vars_.clear();
}

}  // namespace b200net
