// Parameters (env parsing, set-before-get, enum sets, alias prefix) and the environment manager.
#include <cstring>
#include "b200net/assert.h"
#include "b200net/environ.h"
#include "b200net/param.h"
#include "test_util.h"
using namespace b200net;
extern char** environ;

static const char* find(char** env, const char* key) {
  const size_t n = strlen(key);
  for (char** e = env; *e; ++e) if (!strncmp(*e, key, n) && (*e)[n] == '=') return *e + n + 1;
  return nullptr;
}

int main() {
  setenv("OFI_NCCL_T_INT", "42", 1);
  setenv("OFI_NCCL_T_BOOL", "true", 1);
  setenv("OFI_NCCL_T_BAD", "12abc", 1);
  setenv("OFI_NCCL_T_BOTH", "1", 1);
  setenv("B200NET_T_BOTH", "2", 1);
  setenv("OFI_NCCL_T_ENUM", "sendrecv", 1);
  setenv("OFI_NCCL_T_ENUM_BAD", "bogus", 1);
  setenv("OFI_NCCL_T_U64", "0x100", 1);
  Param<int> pi("T_INT", 7);
  Param<bool> pb("T_BOOL", false);
  Param<int> pbad("T_BAD", 5);
  Param<int> pboth("T_BOTH", 0);
  Param<int> pdef("T_UNSET", 9);
  Param<uint64_t> pu("T_U64", 1);
  EnumParam pe("T_ENUM", "RDMA", {"RDMA", "SENDRECV"});
  EnumParam pebad("T_ENUM_BAD", "RDMA", {"RDMA", "SENDRECV"});
  CHECK_EQ(pi.get(), 42); CHECK(pi.source() == ParamSource::ENVIRONMENT);
  CHECK_EQ(pb.get(), true);
  CHECK_EQ(pbad.load_from_env(), -22);
  CHECK_EQ(pbad.get(), 5);                       // malformed value leaves the default
  CHECK_EQ(pboth.get(), 2);                      // own prefix wins over the compatibility prefix
  CHECK_EQ(pdef.get(), 9); CHECK(pdef.source() == ParamSource::DEFAULT);
  CHECK_EQ(pu.get(), 256u);
  CHECK(pe.get() == "sendrecv");
  CHECK_EQ(pebad.load_from_env(), -22); CHECK(pebad.get() == "RDMA");
  // set() works only before the first get()
  Param<int> ps("T_SET", 1);
  CHECK_EQ(ps.set(5), 0); CHECK_EQ(ps.get(), 5); CHECK(ps.source() == ParamSource::API);
  CHECK_EQ(ps.set(6), -22); CHECK_EQ(ps.get(), 5);
  setenv("OFI_NCCL_T_SET2", "3", 1);
  Param<int> ps2("T_SET2", 1);
  CHECK_EQ(ps2.set(8), 0); CHECK_EQ(ps2.get(), 8);  // API beats environment
  CHECK(param_registry().size() >= 10);
  CHECK_EQ(params().eager_max_size.get(), 8192u);
  CHECK_EQ(params().min_stripe_size.get(), 128u * 1024);
  CHECK_THROWS(B200NET_ASSERT_ALWAYS(1 == 2));

  // retired settings: a deprecated one is read with a warning, a removed one fails start-up
  {
    RetiredParam<bool> dep("UNIT_DEPRECATED_SETTING", false, "use something else", false);
    RetiredParam<uint64_t> gone("UNIT_REMOVED_SETTING", 0, "use something else", true);
    CHECK_EQ(dep.load_from_env(), 0);                 // not set: silent
    CHECK_EQ(gone.load_from_env(), 0);
    setenv("B200NET_UNIT_DEPRECATED_SETTING", "1", 1);
    setenv("OFI_NCCL_UNIT_REMOVED_SETTING", "7", 1);  // the reference's prefix counts as well
    dep.reset_for_testing(false);
    gone.reset_for_testing(0);
    CHECK_EQ(dep.load_from_env(), 0);
    CHECK(dep.get());                                 // still honoured
    CHECK_EQ(gone.load_from_env(), -22);
    unsetenv("B200NET_UNIT_DEPRECATED_SETTING");
    unsetenv("OFI_NCCL_UNIT_REMOVED_SETTING");
  }
  // the three settings retired from the reference are known
  CHECK_EQ(params().rdma_min_posted_bounce_buffers.load_from_env(), 0);
  CHECK_EQ(params().endpoint_per_comm.load_from_env(), 0);

  // environment manager: no setenv, fresh array, overwrite semantics
  setenv("KEEP_ME", "old", 1);
  setenv("REPLACE_ME", "old", 1);
  char** before = environ;
  EnvManager& em = EnvManager::instance();
  em.insert_envvar("NEW_VAR", "v1", false);
  em.insert_envvar("NEW_VAR", "v2", false);     // first writer wins
  em.insert_envvar("KEEP_ME", "new", false);    // exists in the process: kept
  em.insert_envvar("REPLACE_ME", "new", true);
  CHECK_EQ(em.pending(), 3u);
  em.update_environment(&environ);
  CHECK(environ != before);
  CHECK(!strcmp(getenv("NEW_VAR"), "v1"));
  CHECK(!strcmp(getenv("KEEP_ME"), "old"));
  CHECK(!strcmp(getenv("REPLACE_ME"), "new"));
  CHECK(!strcmp(find(before, "REPLACE_ME"), "old"));  // the retired array is intact
  CHECK_EQ(em.pending(), 0u);

  TEST_MAIN_END();
}
