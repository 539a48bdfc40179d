// NpKit implementation: buffers, clock alignment, dump files.
#include <mscclpp/npkit/npkit.hpp>

#include <chrono>
#include <fstream>
#include <memory>
#include <mutex>
#include <vector>

#include <cuda_runtime.h>

#include <mscclpp/errors.hpp>

namespace {

struct State {
  int rank = 0;
  bool enabled = false;
  NpKitEvent* gpuEvents = nullptr;                  // kNumGpuEventBuffers * kMaxNumGpuEventsPerBuffer
  NpKitEventCollectContext* gpuContexts = nullptr;  // device array
  std::vector<std::unique_ptr<NpKitEvent[]>> cpuEvents;
  std::vector<uint64_t> cpuHeads;
  uint64_t syncGpuNs = 0, syncCpuNs = 0;
  std::mutex mutex;
};

State& state() {
  static State s;
  return s;
}

__global__ void npkitReadTimer(uint64_t* out) { *out = mscclpp::ptx::globaltimer(); }

uint64_t nowNs() {
  return static_cast<uint64_t>(
      std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::system_clock::now().time_since_epoch()).count());
}

void writeText(const std::string& path, const std::string& text) {
  std::ofstream f(path, std::ios::out | std::ios::trunc);
  f << text;
}

}  // namespace

void NpKit::Init(int rank) {
  State& s = state();
  std::lock_guard<std::mutex> lock(s.mutex);
  if (s.enabled) return;
  s.rank = rank;
  const size_t total = kNumGpuEventBuffers * kMaxNumGpuEventsPerBuffer;
  MSCCLPP_CUDATHROW(cudaMalloc(&s.gpuEvents, total * sizeof(NpKitEvent)));
  MSCCLPP_CUDATHROW(cudaMalloc(&s.gpuContexts, kNumGpuEventBuffers * sizeof(NpKitEventCollectContext)));
  std::vector<NpKitEventCollectContext> ctx(kNumGpuEventBuffers);
  for (uint64_t i = 0; i < kNumGpuEventBuffers; i++) ctx[i] = NpKitEventCollectContext{s.gpuEvents + i * kMaxNumGpuEventsPerBuffer, 0};
  MSCCLPP_CUDATHROW(cudaMemcpy(s.gpuContexts, ctx.data(), ctx.size() * sizeof(ctx[0]), cudaMemcpyHostToDevice));
  s.cpuEvents.clear();
  for (uint64_t i = 0; i < kNumCpuEventBuffers; i++) s.cpuEvents.emplace_back(new NpKitEvent[kMaxNumCpuEventsPerBuffer]);
  s.cpuHeads.assign(kNumCpuEventBuffers, 0);
  // one (device, host) time pair; the host stamp is the middle of the bracket around a synchronous read
  uint64_t* dTimer = nullptr;
  MSCCLPP_CUDATHROW(cudaMalloc(&dTimer, sizeof(uint64_t)));
  npkitReadTimer<<<1, 1>>>(dTimer);  // warm-up: module load must not sit inside the bracket
  MSCCLPP_CUDATHROW(cudaDeviceSynchronize());
  const uint64_t t0 = nowNs();
  npkitReadTimer<<<1, 1>>>(dTimer);
  MSCCLPP_CUDATHROW(cudaDeviceSynchronize());
  const uint64_t t1 = nowNs();
  MSCCLPP_CUDATHROW(cudaMemcpy(&s.syncGpuNs, dTimer, sizeof(uint64_t), cudaMemcpyDeviceToHost));
  MSCCLPP_CUDATHROW(cudaFree(dTimer));
  s.syncCpuNs = t0 + (t1 - t0) / 2;
  s.enabled = true;
}

bool NpKit::Enabled() { return state().enabled; }

NpKitEventCollectContext* NpKit::GetGpuEventCollectContexts() { return state().enabled ? state().gpuContexts : nullptr; }

uint64_t NpKit::GetCpuTimestamp() { return nowNs(); }

void NpKit::CollectCpuEvent(uint8_t type, uint32_t size, uint32_t rsvd, uint64_t timestamp, int channelId) {
  State& s = state();
  if (!s.enabled || channelId < 0 || static_cast<uint64_t>(channelId) >= kNumCpuEventBuffers) return;
  std::lock_guard<std::mutex> lock(s.mutex);
  uint64_t& head = s.cpuHeads[channelId];
  if (head >= kMaxNumCpuEventsPerBuffer) return;
  NpKitEvent& e = s.cpuEvents[channelId][head++];
  e.fields.type = type;
  e.fields.size = size;
  e.fields.rsvd = rsvd;
  e.fields.timestamp = timestamp;
}

void NpKit::Dump(const std::string& dumpDir) {
  State& s = state();
  std::lock_guard<std::mutex> lock(s.mutex);
  if (!s.enabled) return;
  MSCCLPP_CUDATHROW(cudaDeviceSynchronize());
  const std::string suffix = std::to_string(s.rank);
  for (uint64_t i = 0; i < kNumCpuEventBuffers; i++) {
    if (s.cpuHeads[i] == 0) continue;
    std::ofstream f(dumpDir + "/cpu_events_rank_" + suffix + "_channel_" + std::to_string(i), std::ios::out | std::ios::binary);
    f.write(reinterpret_cast<const char*>(s.cpuEvents[i].get()), s.cpuHeads[i] * sizeof(NpKitEvent));
  }
  // both time lines are in nanoseconds: period 1/1e9 s for the host, 1e6 kHz for the device
  writeText(dumpDir + "/cpu_clock_period_num_rank_" + suffix, "1");
  writeText(dumpDir + "/cpu_clock_period_den_rank_" + suffix, "1000000000");
  writeText(dumpDir + "/gpu_clock_rate_rank_" + suffix, "1000000");
  writeText(dumpDir + "/gpu_time_sync_rank_" + suffix, std::to_string(s.syncGpuNs) + " " + std::to_string(s.syncCpuNs));
  std::vector<NpKitEventCollectContext> ctx(kNumGpuEventBuffers);
  MSCCLPP_CUDATHROW(cudaMemcpy(ctx.data(), s.gpuContexts, ctx.size() * sizeof(ctx[0]), cudaMemcpyDeviceToHost));
  std::vector<NpKitEvent> host;
  for (uint64_t i = 0; i < kNumGpuEventBuffers; i++) {
    const uint64_t n = ctx[i].event_buffer_head;
    if (n == 0) continue;
    host.resize(n);
    MSCCLPP_CUDATHROW(cudaMemcpy(host.data(), ctx[i].event_buffer, n * sizeof(NpKitEvent), cudaMemcpyDeviceToHost));
    std::ofstream f(dumpDir + "/gpu_events_rank_" + suffix + "_buf_" + std::to_string(i), std::ios::out | std::ios::binary);
    f.write(reinterpret_cast<const char*>(host.data()), n * sizeof(NpKitEvent));
  }
}

void NpKit::Shutdown() {
  State& s = state();
  std::lock_guard<std::mutex> lock(s.mutex);
  if (!s.enabled) return;
  s.enabled = false;
  (void)cudaFree(s.gpuEvents);
  (void)cudaFree(s.gpuContexts);
  s.gpuEvents = nullptr;
  s.gpuContexts = nullptr;
  s.cpuEvents.clear();
  s.cpuHeads.clear();
}
