// Bindings of the host API (Communicator, connections, registered memory, semaphores, channels, FIFO,
// proxy service, NVLS connection, GPU buffers). Device handles are exposed as raw bytes (`.raw`) so
// Python can pack them into kernel arguments, as the reference's module does
// (python/csrc/{core,semaphore,memory_channel,port_channel,switch_channel,fifo}_py.cpp).
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>

#include <mscclpp/core.hpp>
#include <mscclpp/numa.hpp>
#include <mscclpp/utils.hpp>
#include <mscclpp/fifo.hpp>
#include <mscclpp/gpu_utils.hpp>
#include <mscclpp/memory_channel.hpp>
#include <mscclpp/port_channel.hpp>
#include <mscclpp/semaphore.hpp>
#include <mscclpp/switch_channel.hpp>

#include "bindings.hpp"

namespace py = pybind11;
using namespace mscclpp;

namespace {

template <typename T>
py::bytes rawBytes(const T& v) {
  return py::bytes(reinterpret_cast<const char*>(&v), sizeof(T));
}

template <typename Handle>
void bindHandle(py::module_& m, const char* name) {
  py::class_<Handle>(m, name)
      .def_property_readonly("raw", [](const Handle& h) { return rawBytes(h); })
      .def_property_readonly_static("size", [](py::object) { return sizeof(Handle); });
}

std::vector<char> toVec(const py::bytes& b) {
  std::string s = b;
  return std::vector<char>(s.begin(), s.end());
}

// A device allocation owned by Python: VMM-backed (multicast-bindable) when NVLS is available.
struct RawGpuBuffer {
  explicit RawGpuBuffer(size_t bytes, GpuBufferGranularity granularity = GpuBufferGranularity::MultiCastRecommended)
      : buffer(bytes, granularity) {}
  GpuBuffer<char> buffer;
};

}  // namespace

void registerCoreBindings(py::module_& m) {
  py::enum_<Transport>(m, "Transport")
      .value("Unknown", Transport::Unknown)
      .value("CudaIpc", Transport::CudaIpc)
      .value("IB0", Transport::IB0)
      .value("IB1", Transport::IB1)
      .value("IB2", Transport::IB2)
      .value("IB3", Transport::IB3)
      .value("IB4", Transport::IB4)
      .value("IB5", Transport::IB5)
      .value("IB6", Transport::IB6)
      .value("IB7", Transport::IB7)
      .value("Ethernet", Transport::Ethernet)
      .value("NumTransports", Transport::NumTransports);
  py::class_<TransportFlags>(m, "TransportFlags")
      .def(py::init<>())
      .def(py::init<Transport>())
      .def("has", &TransportFlags::has)
      .def("none", &TransportFlags::none)
      .def("any", &TransportFlags::any)
      .def("count", &TransportFlags::count)
      .def("all", &TransportFlags::all)
      .def("__ior__", [](TransportFlags& a, const TransportFlags& b) { a |= b; return a; })
      .def("__iand__", [](TransportFlags& a, const TransportFlags& b) { a &= b; return a; })
      .def("__or__", [](const TransportFlags& a, const TransportFlags& b) { return a | b; })
      .def("__or__", [](const TransportFlags& a, Transport b) { return a | b; })
      .def("__and__", [](const TransportFlags& a, const TransportFlags& b) { return a & b; })
      .def("__eq__", [](const TransportFlags& a, const TransportFlags& b) { return a == b; });
  py::implicitly_convertible<Transport, TransportFlags>();

  py::enum_<DeviceType>(m, "DeviceType").value("Unknown", DeviceType::Unknown).value("CPU", DeviceType::CPU).value("GPU", DeviceType::GPU);
  py::class_<Device>(m, "Device")
      .def(py::init<>())
      .def(py::init<DeviceType, int>(), py::arg("type"), py::arg("id") = -1)
      .def_readwrite("type", &Device::type)
      .def_readwrite("id", &Device::id);
  py::enum_<EndpointConfig::Ib::Mode>(m, "IbMode")
      .value("Default", EndpointConfig::Ib::Mode::Default)
      .value("Host", EndpointConfig::Ib::Mode::Host)
      .value("HostNoAtomic", EndpointConfig::Ib::Mode::HostNoAtomic);
  py::class_<EndpointConfig::Ib>(m, "EndpointConfigIb")
      .def(py::init<>())
      .def_readwrite("device_index", &EndpointConfig::Ib::deviceIndex)
      .def_readwrite("port", &EndpointConfig::Ib::port)
      .def_readwrite("gid_index", &EndpointConfig::Ib::gidIndex)
      .def_readwrite("max_cq_size", &EndpointConfig::Ib::maxCqSize)
      .def_readwrite("max_cq_poll_num", &EndpointConfig::Ib::maxCqPollNum)
      .def_readwrite("max_send_wr", &EndpointConfig::Ib::maxSendWr)
      .def_readwrite("max_recv_wr", &EndpointConfig::Ib::maxRecvWr)
      .def_readwrite("max_wr_per_send", &EndpointConfig::Ib::maxWrPerSend)
      .def_readwrite("mode", &EndpointConfig::Ib::mode);
  py::class_<EndpointConfig>(m, "EndpointConfig")
      .def(py::init<>())
      .def(py::init<Transport>())
      .def(py::init<Transport, Device, int>(), py::arg("transport"), py::arg("device"), py::arg("max_write_queue_size") = -1)
      .def_readwrite("transport", &EndpointConfig::transport)
      .def_readwrite("device", &EndpointConfig::device)
      .def_readwrite("max_write_queue_size", &EndpointConfig::maxWriteQueueSize)
      .def_readwrite("ib", &EndpointConfig::ib);
  py::implicitly_convertible<Transport, EndpointConfig>();

  py::class_<Endpoint>(m, "Endpoint")
      .def("transport", &Endpoint::transport)
      .def("device", &Endpoint::device)
      .def("host_hash", &Endpoint::hostHash)
      .def("pid_hash", &Endpoint::pidHash)
      .def("max_write_queue_size", &Endpoint::maxWriteQueueSize)
      .def("config", &Endpoint::config)
      .def("serialize", [](const Endpoint& e) {
        auto v = e.serialize();
        return py::bytes(v.data(), v.size());
      })
      .def_static("deserialize", [](py::bytes b) { return Endpoint::deserialize(toVec(b)); });

  py::class_<RegisteredMemory>(m, "RegisteredMemory")
      .def(py::init<>())
      .def("data", [](const RegisteredMemory& r) { return reinterpret_cast<uintptr_t>(r.data()); })
      .def("original_data_ptr", [](const RegisteredMemory& r) { return reinterpret_cast<uintptr_t>(r.originalDataPtr()); })
      .def("size", &RegisteredMemory::size)
      .def("transports", &RegisteredMemory::transports)
      .def("serialize", [](const RegisteredMemory& r) {
        auto v = r.serialize();
        return py::bytes(v.data(), v.size());
      })
      .def_static("deserialize", [](py::bytes b) { return RegisteredMemory::deserialize(toVec(b)); });

  py::class_<Connection>(m, "Connection")
      .def("write",
           [](Connection& c, RegisteredMemory dst, uint64_t dstOffset, RegisteredMemory src, uint64_t srcOffset, uint64_t size) {
             c.write(dst, dstOffset, src, srcOffset, size);
           })
      .def("update_and_sync",
           [](Connection& c, RegisteredMemory dst, uint64_t dstOffset, uintptr_t src, uint64_t newValue) {
             c.updateAndSync(dst, dstOffset, reinterpret_cast<uint64_t*>(src), newValue);
           })
      .def("flush", [](Connection& c, int64_t timeoutUsec) {
        py::gil_scoped_release rel;
        c.flush(timeoutUsec);
      }, py::arg("timeout_usec") = -1)
      .def("transport", &Connection::transport)
      .def("remote_transport", &Connection::remoteTransport)
      .def("local_device", &Connection::localDevice)
      .def("get_max_write_queue_size", &Connection::getMaxWriteQueueSize)
      .def("context", &Connection::context);

  py::class_<Context, std::shared_ptr<Context>>(m, "Context")
      .def_static("create", &Context::create)
      .def("register_memory", [](Context& c, uintptr_t ptr, size_t size, TransportFlags f) {
        return c.registerMemory(reinterpret_cast<void*>(ptr), size, f);
      })
      .def("create_endpoint", &Context::createEndpoint)
      .def("connect", &Context::connect);

  py::class_<std::shared_future<RegisteredMemory>>(m, "RegisteredMemoryFuture").def("get", [](std::shared_future<RegisteredMemory>& f) {
    py::gil_scoped_release rel;
    return f.get();
  });
  py::class_<std::shared_future<Connection>>(m, "ConnectionFuture").def("get", [](std::shared_future<Connection>& f) {
    py::gil_scoped_release rel;
    return f.get();
  });
  py::class_<std::shared_future<Semaphore>>(m, "SemaphoreFuture").def("get", [](std::shared_future<Semaphore>& f) {
    py::gil_scoped_release rel;
    return f.get();
  });

  py::class_<Semaphore>(m, "Semaphore")
      .def(py::init<>())
      .def("local_memory", &Semaphore::localMemory)
      .def("remote_memory", &Semaphore::remoteMemory)
      .def("connection", &Semaphore::connection, py::return_value_policy::reference_internal);

  py::class_<Communicator, std::shared_ptr<Communicator>>(m, "Communicator")
      .def(py::init<std::shared_ptr<Bootstrap>, std::shared_ptr<Context>>(), py::arg("bootstrap"), py::arg("context") = nullptr)
      .def("bootstrap", &Communicator::bootstrap)
      .def("context", &Communicator::context)
      .def("register_memory", [](Communicator& c, uintptr_t ptr, size_t size, TransportFlags f) {
        return c.registerMemory(reinterpret_cast<void*>(ptr), size, f);
      })
      .def("send_memory", &Communicator::sendMemory, py::arg("memory"), py::arg("remote_rank"), py::arg("tag") = 0)
      .def("recv_memory", &Communicator::recvMemory, py::arg("remote_rank"), py::arg("tag") = 0)
      .def("connect", [](Communicator& c, const EndpointConfig& cfg, int remoteRank, int tag) { return c.connect(cfg, remoteRank, tag); },
           py::arg("local_config"), py::arg("remote_rank"), py::arg("tag") = 0)
      .def("connect", [](Communicator& c, const Endpoint& e, int remoteRank, int tag) { return c.connect(e, remoteRank, tag); },
           py::arg("local_endpoint"), py::arg("remote_rank"), py::arg("tag") = 0)
      .def("build_semaphore", &Communicator::buildSemaphore, py::arg("connection"), py::arg("remote_rank"), py::arg("tag") = 0)
      // names of the earlier two-phase API, kept as synonyms: everything is set up when the call returns
      .def("connect_on_setup", [](Communicator& c, int remoteRank, int tag, const EndpointConfig& cfg) { return c.connect(cfg, remoteRank, tag); },
           py::arg("remote_rank"), py::arg("tag"), py::arg("local_config"), py::call_guard<py::gil_scoped_release>())
      .def("send_memory_on_setup", &Communicator::sendMemory, py::arg("memory"), py::arg("remote_rank"), py::arg("tag"))
      .def("recv_memory_on_setup", &Communicator::recvMemory, py::arg("remote_rank"), py::arg("tag"))
      .def("setup", [](Communicator&) {})
      .def("remote_rank_of", &Communicator::remoteRankOf)
      .def("tag_of", &Communicator::tagOf);

  // ------------------------------------------------------------------ semaphores
  bindHandle<Host2DeviceSemaphoreDeviceHandle>(m, "Host2DeviceSemaphoreDeviceHandle");
  bindHandle<MemoryDevice2DeviceSemaphoreDeviceHandle>(m, "MemoryDevice2DeviceSemaphoreDeviceHandle");
  py::class_<Host2DeviceSemaphore, std::shared_ptr<Host2DeviceSemaphore>>(m, "Host2DeviceSemaphore")
      .def(py::init<const Semaphore&>())
      .def(py::init<Communicator&, const Connection&>(), py::call_guard<py::gil_scoped_release>())
      .def("signal", &Host2DeviceSemaphore::signal)
      .def("connection", &Host2DeviceSemaphore::connection, py::return_value_policy::reference_internal)
      .def("device_handle", &Host2DeviceSemaphore::deviceHandle);
  py::class_<Host2HostSemaphore, std::shared_ptr<Host2HostSemaphore>>(m, "Host2HostSemaphore")
      .def(py::init<const Semaphore&>())
      .def(py::init<Communicator&, const Connection&>(), py::call_guard<py::gil_scoped_release>())
      .def("signal", &Host2HostSemaphore::signal)
      .def("connection", &Host2HostSemaphore::connection, py::return_value_policy::reference_internal)
      .def("poll", &Host2HostSemaphore::poll)
      .def("wait", [](Host2HostSemaphore& s, int64_t maxSpin) {
        py::gil_scoped_release rel;
        s.wait(maxSpin);
      }, py::arg("max_spin_count") = 10000000);
  py::class_<MemoryDevice2DeviceSemaphore, std::shared_ptr<MemoryDevice2DeviceSemaphore>>(m, "MemoryDevice2DeviceSemaphore")
      .def(py::init<const Semaphore&>())
      .def(py::init<Communicator&, const Connection&>(), py::call_guard<py::gil_scoped_release>())
      .def("connection", &MemoryDevice2DeviceSemaphore::connection, py::return_value_policy::reference_internal)
      .def("device_handle", &MemoryDevice2DeviceSemaphore::deviceHandle);

  // ------------------------------------------------------------------ channels
  bindHandle<BaseMemoryChannelDeviceHandle>(m, "BaseMemoryChannelDeviceHandle");
  bindHandle<MemoryChannelDeviceHandle>(m, "MemoryChannelDeviceHandle");
  bindHandle<BasePortChannelDeviceHandle>(m, "BasePortChannelDeviceHandle");
  bindHandle<PortChannelDeviceHandle>(m, "PortChannelDeviceHandle");
  bindHandle<SwitchChannelDeviceHandle>(m, "SwitchChannelDeviceHandle");
  bindHandle<FifoDeviceHandle>(m, "FifoDeviceHandle");
  py::class_<BaseMemoryChannel>(m, "BaseMemoryChannel")
      .def(py::init<std::shared_ptr<MemoryDevice2DeviceSemaphore>>())
      .def(py::init<const Semaphore&>())
      .def("device_handle", &BaseMemoryChannel::deviceHandle);
  py::class_<MemoryChannel>(m, "MemoryChannel")
      .def(py::init([](std::shared_ptr<MemoryDevice2DeviceSemaphore> sem, RegisteredMemory dst, RegisteredMemory src, uintptr_t pkt) {
             return MemoryChannel(sem, dst, src, reinterpret_cast<void*>(pkt));
           }),
           py::arg("semaphore"), py::arg("dst"), py::arg("src"), py::arg("packet_buffer") = 0)
      .def(py::init([](const Semaphore& sem, RegisteredMemory dst, RegisteredMemory src, uintptr_t pkt) {
             return MemoryChannel(sem, dst, src, reinterpret_cast<void*>(pkt));
           }),
           py::arg("semaphore"), py::arg("dst"), py::arg("src"), py::arg("packet_buffer") = 0)
      .def("device_handle", &MemoryChannel::deviceHandle);
  py::class_<BasePortChannel>(m, "BasePortChannel").def("device_handle", &BasePortChannel::deviceHandle);
  py::class_<PortChannel>(m, "PortChannel").def("device_handle", &PortChannel::deviceHandle);

  py::class_<ProxyTrigger>(m, "ProxyTrigger").def(py::init<>()).def_readwrite("fst", &ProxyTrigger::fst).def_readwrite("snd", &ProxyTrigger::snd);
  py::class_<Fifo, std::shared_ptr<Fifo>>(m, "Fifo")
      .def(py::init<int>(), py::arg("size") = DEFAULT_FIFO_SIZE)
      .def("poll", &Fifo::poll)
      .def("pop", &Fifo::pop)
      .def("size", &Fifo::size)
      .def("consumed", &Fifo::consumed)
      .def("push_from_host", &Fifo::pushFromHost)
      .def("device_handle", &Fifo::deviceHandle);
  py::class_<ProxyService, std::shared_ptr<ProxyService>>(m, "ProxyService")
      .def(py::init<int>(), py::arg("fifo_size") = DEFAULT_FIFO_SIZE)
      .def("start_proxy", &ProxyService::startProxy, py::arg("blocking") = false)
      .def("stop_proxy", &ProxyService::stopProxy)
      .def("build_and_add_semaphore", &ProxyService::buildAndAddSemaphore, py::call_guard<py::gil_scoped_release>())
      .def("add_semaphore", [](ProxyService& s, const Semaphore& sem) { return s.addSemaphore(sem); })
      .def("add_memory", &ProxyService::addMemory)
      .def("next_memory_id", &ProxyService::nextMemoryId, py::arg("count") = 1)
      .def("semaphore", &ProxyService::semaphore)
      .def("base_port_channel", &ProxyService::basePortChannel)
      .def("port_channel", &ProxyService::portChannel);

  py::class_<SwitchChannel>(m, "SwitchChannel")
      .def("device_handle", &SwitchChannel::deviceHandle)
      .def("get_device_ptr", [](SwitchChannel& c) { return reinterpret_cast<uintptr_t>(c.getDevicePtr()); })
      .def("get_mc_ptr", [](SwitchChannel& c) { return reinterpret_cast<uintptr_t>(c.getMcPtr()); });
  py::class_<NvlsConnection, std::shared_ptr<NvlsConnection>>(m, "NvlsConnection")
      .def_static("get_multicast_min_granularity", &NvlsConnection::getMultiCastMinGranularity)
      .def("bind_allocated_memory", [](NvlsConnection& c, uintptr_t ptr, size_t size) {
        py::gil_scoped_release rel;
        return c.bindAllocatedMemory(reinterpret_cast<void*>(ptr), size);
      })
      .def("capacity", &NvlsConnection::capacity);
  m.def("connect_nvls_collective", [](std::shared_ptr<Communicator> comm, std::vector<int> ranks, size_t bytes) {
    py::gil_scoped_release rel;
    return connectNvlsCollective(comm, ranks, bytes);
  });

  // ------------------------------------------------------------------ buffers
  m.def("get_host_name", &getHostName, py::arg("maxlen"), py::arg("delim"));
  py::enum_<GpuBufferGranularity>(m, "GpuBufferGranularity")
      .value("MultiCastMinimum", GpuBufferGranularity::MultiCastMinimum)
      .value("MultiCastRecommended", GpuBufferGranularity::MultiCastRecommended);
  {
    py::module_ numa = m.def_submodule("numa", "NUMA placement helpers");
    numa.def("get_device_numa_node", &getDeviceNumaNode, py::arg("device_id"));
    numa.def("get_numa_node_cpus", &getNumaNodeCpus, py::arg("node"));
    numa.def("numa_bind", &numaBind, py::arg("node"));
    numa.def("parse_cpu_list", &parseCpuList, py::arg("text"));
  }
  py::class_<RawGpuBuffer, std::shared_ptr<RawGpuBuffer>>(m, "RawGpuBuffer")
      .def(py::init<size_t, GpuBufferGranularity>(), py::arg("nbytes"),
           py::arg("granularity") = GpuBufferGranularity::MultiCastRecommended)
      .def("data", [](RawGpuBuffer& b) { return reinterpret_cast<uintptr_t>(b.buffer.data()); })
      .def("bytes", [](RawGpuBuffer& b) { return b.buffer.bytes(); })
      .def("nelems", [](RawGpuBuffer& b) { return b.buffer.nelems(); })
      .def("device_id", [](RawGpuBuffer& b) { return b.buffer.deviceId(); });
}
