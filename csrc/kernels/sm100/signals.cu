// Device-side gates between streams, stages and processes, each with a bounded wait:
//   kern_hold   wait until *counter >= want (an arrival count another GPU's copy or a host thread advances);
//               gives up after timeout_ns, sets the error word and lets the program run on (the host sees the error)
//   kern_mark   publish a sequence number to a (pinned or peer) word after everything before it in the stream
//   kern_lanes_step / kern_lanes_join   test kernels for the runtime's lanes: a timed busy step, and a join that
//               adds what the steps wrote
// Reference counterparts: crates/kern-runtime/src/exec.rs:135-164 (hold / flag PTX), tools/kernels-src/lanes.cu:19-28.
#include "common.cuh"

using namespace kern;

extern "C" __global__ void kern_hold(const unsigned long long* counter, unsigned long long want, long long timeout_ns,
                                     int* err, int code) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const uint64_t t0 = globaltimer_ns();
  while (true) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(counter) : "memory");
    if (v >= want) return;
    if ((long long)(globaltimer_ns() - t0) > timeout_ns) {
      set_error(err, code);
      return;
    }
    __nanosleep(200);
  }
}

extern "C" __global__ void kern_mark(unsigned long long* word, unsigned long long value) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(word), "l"(value) : "memory");
}

// Adds 1 to counter (an arrival), system scope: what a pushing side runs after its copy.
extern "C" __global__ void kern_arrive(unsigned long long* counter) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  __threadfence_system();
  atomicAdd_system(counter, 1ull);
}

extern "C" __global__ void kern_lanes_step(float* out, int index, float value, long long busy_ns) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const uint64_t t0 = globaltimer_ns();
  const long long limit = busy_ns < 50000000ll ? busy_ns : 50000000ll;      // never longer than 50 ms
  while ((long long)(globaltimer_ns() - t0) < limit) __nanosleep(500);
  out[index] = value;
}

extern "C" __global__ void kern_lanes_join(const float* in, float* out, int n) {
  pdl_wait();
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  float s = 0.f;
  for (int i = 0; i < n; ++i) s += in[i];
  out[0] = s;
}
