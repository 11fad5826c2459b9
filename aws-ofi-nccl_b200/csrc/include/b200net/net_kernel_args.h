// Argument block of the plugin's batched copy kernel, shared by the device code, the host side
// that fills it and the stand-in driver of the CPU tests. Plain C layout, passed by value as the
// kernel's one parameter (it fits the parameter space: 16 jobs of 56 bytes).
#pragma once

#define B200NET_BATCH_MAX_JOBS 16

struct B200NetBatchJob {
  unsigned char* dst;
  const unsigned char* src;
  unsigned long long bytes;
  unsigned int* counter;           // device word of the job's completion slot: counts the CTAs that finished
  unsigned long long* flag;        // completion word in pinned host memory
  unsigned long long flag_value;   // written there by the CTA that finishes last (| 1 << 63: a wait ran out)
  unsigned int cta_begin;          // first CTA of the grid that works on this job
  unsigned int ctas;               // how many CTAs do
};

struct B200NetBatchArgs {
  struct B200NetBatchJob job[B200NET_BATCH_MAX_JOBS];
  unsigned long long wait_limit_ns;
  unsigned int njobs;
  unsigned int bulk_mask;          // bit j: job j may use the bulk-copy path (16-byte aligned, device source)
};
