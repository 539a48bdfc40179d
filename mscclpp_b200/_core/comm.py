"""`CommGroup`: bootstrap + communicator + the usual channel-construction helpers in one object
(reference: python/mscclpp/_core/comm.py:30-282)."""
from __future__ import annotations

import pickle
from typing import Dict, Optional

from . import native as _loader

__all__ = ["CommGroup"]


def _ptr_and_bytes(tensor):
    if hasattr(tensor, "data_ptr"):  # torch
        return tensor.data_ptr(), tensor.numel() * tensor.element_size()
    if hasattr(tensor, "__cuda_array_interface__"):
        return tensor.__cuda_array_interface__["data"][0], tensor.size * tensor.itemsize
    return tensor.ctypes.data, tensor.size * tensor.itemsize  # numpy


class CommGroup:
    def __init__(self, mpi_comm=None, torch_group=None, interfaceIpPortTrio: str = "", rank: Optional[int] = None,
                 size: Optional[int] = None):
        n = _loader.load()
        if interfaceIpPortTrio == "" and (mpi_comm is not None or torch_group is not None):
            if mpi_comm is not None:
                rank, size = mpi_comm.Get_rank(), mpi_comm.Get_size()
            else:
                rank, size = torch_group.rank(), torch_group.size()
            self.bootstrap = n.TcpBootstrap.create(rank, size)
            uniq_id = self.bootstrap.create_unique_id() if rank == 0 else None
            if mpi_comm is not None:
                uniq_id = mpi_comm.bcast(uniq_id, 0)
            else:
                import torch
                import torch.distributed as dist

                box = [pickle.dumps(uniq_id)] if rank == 0 else [None]
                dist.broadcast_object_list(box, src=dist.get_global_rank(torch_group, 0), group=torch_group,
                                           device=torch.device("cpu") if dist.get_backend(torch_group) == "gloo" else None)
                uniq_id = pickle.loads(box[0])
            self.bootstrap.initialize(uniq_id)
        elif interfaceIpPortTrio != "":
            assert rank is not None and size is not None and rank >= 0 and size >= 1
            self.bootstrap = n.TcpBootstrap.create(rank, size)
            self.bootstrap.initialize(interfaceIpPortTrio)
        else:
            raise RuntimeError("Either the interface or mpi_group need to be specified")
        self.communicator = n.Communicator(self.bootstrap)
        self.my_rank = self.bootstrap.get_rank()
        self.nranks = self.bootstrap.get_n_ranks()
        self.nranks_per_node = self.bootstrap.get_n_ranks_per_node()
        self.nranks_per_ipc_domain = self.bootstrap.get_n_ranks_per_ipc_domain()
        self.ipc_domain_n_ranks = self.nranks_per_ipc_domain

    def barrier(self):
        self.bootstrap.barrier()

    def send(self, tensor, peer: int, tag: int):
        self.bootstrap.send(bytes(memoryview(tensor).cast("B")), peer, tag)

    def recv(self, tensor, peer: int, tag: int):
        data = self.bootstrap.recv(peer, tag)
        memoryview(tensor).cast("B")[:] = data

    def my_ib_device(self, local_rank: int):
        n = _loader.load()
        assert 0 <= local_rank < 8, "only 8 IB devices are addressable"
        return getattr(n.Transport, f"IB{local_rank}")

    def make_connection(self, all_ranks, endpoints, use_switch: bool = False) -> Dict[int, object]:
        n = _loader.load()
        if isinstance(endpoints, n.Transport):
            endpoints = n.EndpointConfig(endpoints)
        elif isinstance(endpoints, dict):
            endpoints = {k: n.EndpointConfig(v) if isinstance(v, n.Transport) else v for k, v in endpoints.items()}
        futures = {}
        for rank in all_ranks:
            endpoint = endpoints[rank] if isinstance(endpoints, dict) else endpoints
            if endpoint.transport == n.Transport.CudaIpc and use_switch:
                return n.connect_nvls_collective(self.communicator, list(all_ranks), 2**30)
            futures[rank] = self.communicator.connect(endpoint, rank)
        return {rank: f.get() for rank, f in futures.items()}

    def register_local_memory(self, tensor, connections):
        n = _loader.load()
        flags = n.TransportFlags()
        for rank in connections:
            flags |= connections[rank].transport()
        ptr, nbytes = _ptr_and_bytes(tensor)
        return self.communicator.register_memory(ptr, nbytes, flags)

    def _register_memory_with_connections(self, memory, connections):
        out = {self.my_rank: memory}
        futures = {}
        for rank in connections:
            self.communicator.send_memory(memory, rank)
            futures[rank] = self.communicator.recv_memory(rank)
        for rank in connections:
            out[rank] = futures[rank].get()
        return out

    def register_tensor_with_connections(self, tensor, connections):
        return self._register_memory_with_connections(self.register_local_memory(tensor, connections), connections)

    def make_semaphores(self, connections):
        futures = {rank: self.communicator.build_semaphore(connections[rank], rank) for rank in connections}
        return {rank: f.get() for rank, f in futures.items()}

    def make_memory_channels(self, tensor, connections):
        n = _loader.load()
        semaphores = self.make_semaphores(connections)
        memories = self.register_tensor_with_connections(tensor, connections)
        return {rank: n.MemoryChannel(semaphores[rank], memories[rank], memories[self.my_rank]) for rank in connections}

    def make_memory_channels_with_scratch(self, tensor, registeredScratchBuffer, connections):
        n = _loader.load()
        semaphores = self.make_semaphores(connections)
        memories = self._register_memory_with_connections(registeredScratchBuffer, connections)
        ptr, nbytes = _ptr_and_bytes(tensor)
        local = self.communicator.register_memory(ptr, nbytes, n.TransportFlags())
        scratch_ptr = registeredScratchBuffer.data()
        return {rank: n.MemoryChannel(semaphores[rank], memories[rank], local, scratch_ptr) for rank in connections}

    def make_port_channels(self, proxy_service, tensor, connections):
        semaphores = self.make_semaphores(connections)
        memories = self.register_tensor_with_connections(tensor, connections)
        memory_ids = {rank: proxy_service.add_memory(memories[rank]) for rank in memories}
        semaphore_ids = {rank: proxy_service.add_semaphore(semaphores[rank]) for rank in semaphores}
        return {rank: proxy_service.port_channel(semaphore_ids[rank], memory_ids[rank], memory_ids[self.my_rank]) for rank in semaphores}

    def make_port_channels_with_scratch(self, proxy_service, tensor, registeredScratchBuffer, connections):
        local = self.register_local_memory(tensor, connections)
        semaphores = self.make_semaphores(connections)
        memories = self._register_memory_with_connections(registeredScratchBuffer, connections)
        memory_ids = {}
        for rank in memories:
            memory_ids[rank] = proxy_service.add_memory(local if rank == self.my_rank else memories[rank])
        semaphore_ids = {rank: proxy_service.add_semaphore(semaphores[rank]) for rank in semaphores}
        return {rank: proxy_service.port_channel(semaphore_ids[rank], memory_ids[rank], memory_ids[self.my_rank]) for rank in semaphores}

    def register_semaphore_with_proxy(self, proxy_service, connections):
        semaphores = self.make_semaphores(connections)
        return {rank: proxy_service.base_port_channel(proxy_service.add_semaphore(semaphores[rank])) for rank in semaphores}

    def register_memory_with_proxy(self, proxy_service, tensor, connections):
        memories = self.register_tensor_with_connections(tensor, connections)
        return {rank: proxy_service.add_memory(memories[rank]) for rank in memories}
