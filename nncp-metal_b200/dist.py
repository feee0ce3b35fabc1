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


class ShardedCodec:
    """encode_file / decode_file of a job whose streams are sharded over the ranks of `group`
    (the block walk of nncp.c:2968-3147 with the coder on rank 0).

    Every rank runs the model on its own streams.  What the range coder needs crosses ranks once
    per segment when encoding (each rank's coder-ready prob0 paths, gathered on rank 0 and coded
    there in (t, global stream) order, as the single-process loop does) and once per symbol step
    when decoding (each rank's prob0 trees to rank 0, the decoded symbols back to everyone: a
    decoder learns its next input only from the coder).  Gradients are summed over ranks by
    `step.reduce_gradients()` or inside the model's backward pass, then every rank updates.

    The sum over ranks has an order that depends on their number, so the header records it
    (version 3) and `decompress` refuses a file coded by a different number of ranks.

    `model` provides reset, set_lr, eval(output_index, ids), eval_end, eval_gradient, update and
    either coder_paths / coder_trees (prob0 values computed by the model) or, when it has neither,
    probability tables through eval's return value (the CPU oracle in the tests).  All ranks pass
    the same `symbols`; rank 0 returns the coded bytes, the others None.
    """

    def __init__(self, host, model, model_params, step, group=None, device="cpu"):
        import torch
        self.host, self.m, self.p, self.step, self.group = host, model, model_params, step, group
        self.device = torch.device(device)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.B, self.T, self.V = model_params.n_streams, model_params.seg_len, model_params.n_symbols
        self.Bt = self.B * self.world
        self.ready = hasattr(model, "coder_paths") and self.V > 1    # any alphabet: a power of two or not
        self.L = host.library()

    # ---- plumbing
    def _gather0(self, arr):
        """[...] per rank -> [world, ...] on rank 0 (None elsewhere)."""
        import numpy as np
        import torch
        if self.world == 1:
            return arr[None]
        t = torch.from_numpy(np.ascontiguousarray(arr).view(np.uint8).reshape(-1)).to(self.device)
        out = [torch.empty_like(t) for _ in range(self.world)] if self.rank == 0 else None
        dist.gather(t, out, dst=0, group=self.group)
        if self.rank != 0:
            return None
        return np.stack([o.cpu().numpy().view(arr.dtype).reshape(arr.shape) for o in out])

    def _bcast(self, arr):
        import torch
        if self.world == 1:
            return arr
        t = torch.from_numpy(arr).to(self.device)
        dist.broadcast(t, src=0, group=self.group)
        return t.cpu().numpy()

    @staticmethod
    def _layout(block_len, Bt):
        stride, rem = divmod(block_len, Bt)
        return stride, rem

    def _take(self, block, stride, rem, pos):
        """Symbols at stream position `pos` of every stream (0 where the stream has none)."""
        import numpy as np
        b = np.arange(self.Bt)
        ok = (pos >= 0) & (pos < stride + (b < rem))
        idx = stride * b + np.minimum(b, rem) + pos
        out = np.zeros(self.Bt, np.int32)
        out[ok] = block[idx[ok]]
        return out

    def _put(self, block, stride, rem, pos, syms, n_active):
        import numpy as np
        b = np.arange(n_active)
        block[stride * b + np.minimum(b, rem) + pos] = syms[:n_active]

    def _mine(self, a):
        return a[..., self.rank * self.B:(self.rank + 1) * self.B]

    def _lr(self, fp, step_no):
        import ctypes as C
        return self.L.nch_interp(C.byref(fp.lr), step_no)

    # ---- encode
    def _encode_rows(self, enc, nt, targets_all, limit_t, limit_b):
        """Rows [0, nt) of the forward pass just evaluated: gather what the coder needs, code on rank 0."""
        import ctypes as C
        import numpy as np
        tg = np.ascontiguousarray(self._mine(targets_all)[:nt])
        if self.ready:
            mine = self.m.coder_paths(0, nt, tg).reshape(nt, self.B, -1)
        else:
            mine = np.ascontiguousarray(self.m_probs[:nt])
        g = self._gather0(mine)
        if self.rank != 0:
            return
        rows = np.ascontiguousarray(np.moveaxis(g, 0, 1).reshape(nt, self.Bt, -1))   # [t][global stream][...]
        for t in range(nt):
            n_act = self.Bt if t < limit_t else (limit_b if t == limit_t else 0)
            if n_act <= 0:
                continue
            syms = np.ascontiguousarray(targets_all[t, :n_act], np.int32)
            if self.ready:
                r = np.ascontiguousarray(rows[t, :n_act])
                assert r.shape[-1] == self.L.nch_tree_depth(self.V)
                self.L.nch_write_sym_paths_any(enc, r.ctypes.data_as(C.c_void_p), self.V, syms.ctypes.data_as(C.c_void_p), n_act)
            else:
                for b in range(n_act):
                    r = np.ascontiguousarray(rows[t, b], np.float32)
                    self.L.nch_write_sym(enc, r.ctypes.data_as(C.c_void_p), self.V, int(syms[b]))

    def _eval(self, oi, ids_all):
        import numpy as np
        out = self.m.eval(oi, np.ascontiguousarray(self._mine(ids_all)), **({"read": False} if self.ready else {}))
        if not self.ready:
            self.m_probs = out     # [T or 1][B][V]

    def _train(self, fp, targets_all, train_step):
        import numpy as np
        self.m.set_lr(self._lr(fp, train_step))
        self.m.eval_gradient(np.ascontiguousarray(self._mine(targets_all)))
        self.step.reduce_gradients()
        self.m.update()

    def compress(self, fp, symbols):
        import ctypes as C
        import numpy as np
        if fp.retrain_period:
            raise ValueError("the retrain pass between blocks is single-process (nch_compress)")
        fp.n_ranks = self.world
        fp.model.n_streams = self.Bt     # the header's batch_size is the job's
        symbols = np.ascontiguousarray(symbols, np.uint16)
        n, T, Bt = symbols.size, self.T, self.Bt
        enc = self.L.nch_enc_new() if self.rank == 0 else None
        pos, train_step = 0, 0
        while pos < n:
            bl = self.L.nch_next_block_len(C.byref(fp), pos, n - pos)
            block = symbols[pos:pos + bl].astype(np.int32)
            stride, rem = self._layout(bl, Bt)
            self.m.reset()
            sp = 0
            while sp + T <= stride:
                ids = np.stack([self._take(block, stride, rem, sp + t - 1) for t in range(T)])
                tg = np.stack([self._take(block, stride, rem, sp + t) for t in range(T)])
                self._eval(-1, ids)
                self._encode_rows(enc, T, tg, T, 0)
                self._train(fp, tg, train_step)
                train_step += 1
                sp += T
            tail2 = stride - sp
            tail1 = tail2 + (rem != 0)
            if tail1 > 0:
                ids = np.zeros((T, Bt), np.int32)
                tg = np.zeros((T, Bt), np.int32)
                for t in range(tail1):
                    ids[t] = self._take(block, stride, rem, sp + t - 1)
                    tg[t] = self._take(block, stride, rem, sp + t)
                self._eval(-1, ids)
                self._encode_rows(enc, tail1, tg, tail2, rem)
                getattr(self.m, "eval_end", lambda: None)()   # a model without step state has nothing to end
            pos += bl
        if self.rank != 0:
            return None
        out = C.c_void_p()
        plen = self.L.nch_enc_finish(enc, C.byref(out))
        payload = C.string_at(out.value, plen) if plen else b""
        self.L.nch_enc_free(enc)
        return self.host.header_bytes(fp, n) + payload

    # ---- decode
    def _decode_step(self, dec, t, ids_all, limit_t, limit_b):
        """One symbol of every stream: trees (or tables) to rank 0, symbols back."""
        import ctypes as C
        import numpy as np
        self._eval(t, ids_all)
        mine = self.m.coder_trees(t, 1) if self.ready else np.ascontiguousarray(self.m_probs[0])
        g = self._gather0(mine)
        syms = np.zeros(self.Bt, np.int32)
        n_act = self.Bt if t < limit_t else (limit_b if t == limit_t else 0)
        if self.rank == 0 and n_act > 0:
            rows = np.ascontiguousarray(g.reshape(self.Bt, -1)[:n_act])
            if self.ready:
                self.L.nch_read_sym_trees(dec, rows.ctypes.data_as(C.c_void_p), self.V, n_act, syms.ctypes.data_as(C.c_void_p))
            else:
                for b in range(n_act):
                    r = np.ascontiguousarray(rows[b], np.float32)
                    syms[b] = self.L.nch_read_sym(dec, r.ctypes.data_as(C.c_void_p), self.V)
        return self._bcast(syms), n_act

    def decompress(self, data):
        import ctypes as C
        import numpy as np
        fp, n, used = self.host.read_header(data)
        if max(fp.n_ranks, 1) != self.world:
            raise ValueError(f"the file was coded by {max(fp.n_ranks, 1)} rank(s); {self.world} cannot decode it")
        if fp.model.n_streams != self.Bt:
            raise ValueError(f"the file has {fp.model.n_streams} streams, this job {self.Bt}")
        if fp.retrain_period:
            raise ValueError("the file was coded with a retrain pass between blocks: single-process (nch_decompress)")
        payload = data[used:]
        buf = C.create_string_buffer(payload, max(len(payload), 1))
        dec = self.L.nch_dec_new(buf, len(payload)) if self.rank == 0 else None
        out = np.zeros(n, np.uint16)
        T, Bt = self.T, self.Bt
        pos, train_step = 0, 0
        while pos < n:
            bl = self.L.nch_next_block_len(C.byref(fp), pos, n - pos)
            block = np.zeros(bl, np.int32)
            stride, rem = self._layout(bl, Bt)
            self.m.reset()
            sp = 0
            while sp + T <= stride:
                ids = np.zeros((T, Bt), np.int32)
                tg = np.zeros((T, Bt), np.int32)
                for t in range(T):
                    ids[t] = self._take(block, stride, rem, sp + t - 1)
                    tg[t], _ = self._decode_step(dec, t, ids, T, 0)
                    self._put(block, stride, rem, sp + t, tg[t], Bt)
                self._train(fp, tg, train_step)
                train_step += 1
                sp += T
            tail2 = stride - sp
            tail1 = tail2 + (rem != 0)
            if tail1 > 0:
                ids = np.zeros((T, Bt), np.int32)
                for t in range(tail1):
                    ids[t] = self._take(block, stride, rem, sp + t - 1)
                    s, n_act = self._decode_step(dec, t, ids, tail2, rem)
                    self._put(block, stride, rem, sp + t, s, n_act)
                getattr(self.m, "eval_end", lambda: None)()   # a model without step state has nothing to end
            out[pos:pos + bl] = block
            pos += bl
        if dec:
            self.L.nch_dec_free(dec)
        return out
