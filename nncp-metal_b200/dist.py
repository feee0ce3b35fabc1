"""Stream sharding over ranks (one process per GPU, torch.distributed for the plumbing).

NNCP's parallel streams are independent through forward, backward, memory and K/V state
(mem_h has a stream axis, nncp.c:503-505); they meet only in the gradient of the shared
weights, because the loss is one sum over all T*B positions (nncp.c:1173-1175).  Rank r owns
streams [r*B/N, (r+1)*B/N); after the backward pass the flat fp32 gradient buffers are summed
over ranks (one all-reduce, fixed N and algorithm => every rank gets the same bits), then every
rank applies the same optimizer step to its replica of the weights.
"""
import torch.distributed as dist


def stream_slice(rank, world, n_streams_total):
    """Columns of the [T, B] id / target arrays that rank `rank` owns."""
    if n_streams_total % world:
        raise ValueError(f"{n_streams_total} streams do not divide over {world} ranks")
    per = n_streams_total // world
    return slice(rank * per, (rank + 1) * per)


class ShardedStep:
    """One train step of a stream shard.  `model` has the plugin verbs (eval, eval_gradient,
    update or their *_dev forms); `grads` is a torch tensor aliasing the model's flat gradient
    buffer.  The model must have been created with n_streams_total = the job's stream count so
    that its loss scale is 1/(T*B_total)."""

    def __init__(self, model, grads, world=None, group=None):
        self.model, self.grads, self.group = model, grads, group
        self.world = world if world is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)

    def reduce_gradients(self):
        if getattr(self.model, "has_comm", False):
            return  # the library already summed them, layer by layer, during the backward pass
        if self.world > 1:
            dist.all_reduce(self.grads, op=dist.ReduceOp.SUM, group=self.group)

    def step_host(self, ids, targets):
        self.model.eval(-1, ids)
        loss = self.model.eval_gradient(targets)
        self.reduce_gradients()
        self.model.update()
        return loss

    def fused(self):
        """The optimizer may run inside the backward pass when nobody has to sum gradients after it."""
        import os
        if not hasattr(self.model, "eval_gradient_update_dev"):
            return False
        env = os.environ.get("NNCU_FUSED_UPDATE")
        if env is not None:
            return env == "1" and (self.world == 1 or getattr(self.model, "has_comm", False))
        # measured on the c2 step: 1 GPU 2.897 ms fused against 2.889 ms separate; 2 GPUs (update queued
        # behind each layer's all-reduce) 2.470 ms against 2.493 ms
        return self.world > 1 and getattr(self.model, "has_comm", False)

    def step_device(self, ids_ptr, targets_ptr):
        self.model.eval_dev(-1, ids_ptr)
        if self.fused():
            self.model.eval_gradient_update_dev(targets_ptr)
            self.model.memory_shift()
            return
        self.model.eval_gradient_dev(targets_ptr)
        self.reduce_gradients()
        self.model.update()


class CudaArray:
    """Device memory owned by the C library, exposed through __cuda_array_interface__ so that
    torch can alias it (torch.as_tensor) for the NCCL all-reduce without a copy."""

    def __init__(self, ptr, n_floats):
        self.__cuda_array_interface__ = {"shape": (int(n_floats),), "typestr": "<f4",
                                         "data": (int(ptr), False), "version": 2}


def attach_library_comm(model, lib, rank, world, device):
    """Gives `model` an NCCL communicator of its own (id made on rank 0, broadcast with
    torch.distributed), so that the gradient exchange runs inside the backward pass."""
    import ctypes as C
    import torch
    buf = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        raw = C.create_string_buffer(128)
        if lib.nncu_comm_unique_id(raw) != 0:
            raise RuntimeError(lib.nncu_last_error().decode())
        buf = torch.frombuffer(bytearray(raw.raw), dtype=torch.uint8).clone()
    buf = buf.to(device)
    dist.broadcast(buf, src=0)
    model.comm_init(world, rank, bytes(buf.cpu().numpy().tobytes()))
