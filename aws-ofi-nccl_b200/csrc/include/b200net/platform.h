// Platform layer: per-machine knowledge (latency to advertise, NCCL environment defaults, default
// protocol, rail ordering, device GUIDs, error hints). Several implementations register with the
// manager; the one with the highest priority that recognises the machine wins, unless PLATFORM
// forces one by name (reference: include/nccl_ofi_platform.h:37-176, src/platform-aws.cpp).
#pragma once
#include <cstdint>
#include <memory>
#include <regex>
#include <string>
#include <utility>
#include <vector>

namespace b200net {

struct TopoGpu;

class Platform {
 public:
  virtual ~Platform() = default;
  virtual const char* get_name() const = 0;
  virtual int get_priority() const = 0;         // <0: does not apply to this machine
  virtual int init(std::string* provider_filter) { (void)provider_filter; return 0; }
  // Order the rails (copy channels) of one GPU; default keeps the order.
  virtual void sort_rails(std::vector<int>& rails) { (void)rails; }
  // Points NCCL's tuner loader at the shared object this code lives in (unless the user named a
  // tuner, or B200NET_TUNER_SELF_REGISTER=0): the library carries the tuner tables next to the net
  // plugin, and NCCL only looks for a tuner where NCCL_TUNER_PLUGIN says
  // (reference: src/platform-aws.cpp:577-648). Returns the path that was published, "" if none.
  std::string register_tuner() const;
  virtual uint64_t device_get_guid(int dev_index) const;
  // A human-actionable hint for an error code seen on the completion path ("" if none).
  virtual std::string log_error_hint(int err) const { (void)err; return ""; }
  virtual float latency_us() const { return 0.f; }
  virtual const char* default_protocol() const { return ""; }
  virtual bool gdaki_capable() const { return false; }
  virtual std::vector<std::pair<std::string, std::string>> nccl_env() const { return {}; }
};

class PlatformDefault : public Platform {
 public:
  const char* get_name() const override { return "Default"; }
  int get_priority() const override { return 0; }
};

// One 8-GPU NVSwitch box with Blackwell GPUs (any vendor chassis).
class PlatformB200 : public Platform {
 public:
  explicit PlatformB200(bool detected) : detected_(detected) {}
  const char* get_name() const override { return "B200"; }
  int get_priority() const override { return detected_ ? 100 : -1; }
  int init(std::string* provider_filter) override;
  float latency_us() const override { return 2.0f; }   // NVLink put+signal, not a NIC round trip
  const char* default_protocol() const override { return "RDMA"; }
  bool gdaki_capable() const override { return true; }
  std::vector<std::pair<std::string, std::string>> nccl_env() const override;
  std::string log_error_hint(int err) const override;
  // Ascending rail ids, whatever order discovery produced: rail i of a sender is the stream and
  // completion ring that rail i of its receiver expects (reference: the cloud platform sorts a
  // group's NICs by their virtual-function index for the same reason, src/platform-aws.cpp sort_rails).
  void sort_rails(std::vector<int>& rails) override;

 private:
  bool detected_;
};

// Cloud instance table: name / regex -> settings (kept so that tools that force a product name,
// such as the tuner inspection CLI, see the same decisions per instance type as before).
struct InstanceEntry {
  const char* name;
  const char* regex;       // null: exact name match
  const char* topology;    // static topology file name or null
  bool dup_conns;
  float latency_us;
  bool gdr_required;
  const char* default_protocol;
  bool gdaki;              // kernel-initiated GIN offered
  std::vector<std::pair<std::string, std::string>> env;
};
const std::vector<InstanceEntry>& instance_table();
const InstanceEntry* find_instance(const std::string& product_name);

class PlatformCloud : public Platform {
 public:
  explicit PlatformCloud(const InstanceEntry* e) : e_(e) {}
  const char* get_name() const override { return "AWS"; }
  int get_priority() const override { return e_ ? 50 : -1; }
  float latency_us() const override { return e_ ? e_->latency_us : 0.f; }
  const char* default_protocol() const override { return e_ ? e_->default_protocol : ""; }
  bool gdaki_capable() const override { return e_ && e_->gdaki; }
  std::vector<std::pair<std::string, std::string>> nccl_env() const override;
  const InstanceEntry* entry() const { return e_; }

 private:
  const InstanceEntry* e_;
};

class PlatformManager {
 public:
  static PlatformManager& instance();
  void register_platform(std::unique_ptr<Platform> p);
  void register_all_platforms();  // Default, B200 (if detected), cloud table (if the product name matches)
  // Highest priority >= 0, or the one named by the PLATFORM parameter. Never null after registration.
  Platform* get_platform();
  void clear_for_testing();

 private:
  std::vector<std::unique_ptr<Platform>> platforms_;
  Platform* chosen_ = nullptr;
};

}  // namespace b200net
