"""Tensor-parallel GEMMs fused with their collective (``kernels/csrc/gemm_comm.cu``).

``FusedGemmContext`` owns what the two kernels share between the ranks of one model-parallel group: the signal pad,
two gathered-operand buffers and two staging buffers (alternating by call parity) in IPC-mapped symmetric memory, the
call counter and the status word that a bounded wait raises.

    all_gather_gemm(x_rows, w)        C[world*Ms, N] = gather(x_rows) @ w           (column-parallel forward)
    gemm_reduce_scatter(a, w)         out[Ms, N]     = reduce_scatter(a @ w)        (row-parallel forward)

``ColumnParallelLinear`` / ``RowParallelLinear`` are the autograd pairs of a sequence-parallel transformer block:
activations between blocks are sharded over rows (tokens), the first projection gathers them inside its GEMM and the
second one scatters the reduced result inside its GEMM; their backward passes are the mirror images.  Weight gradients
use the plain tcgen05 GEMM on the gathered operand that the fused kernel already brought into local memory.

The reference runs sharded layers through GSPMD on its JAX backend only (keras/src/backend/jax/distribution_lib.py:32-106).
"""

import ctypes

import torch

from keras_b200.kernels import gemm as kgemm
from keras_b200.kernels import ops as kops
from keras_b200.parallel import collectives, process_groups
from keras_b200.parallel.symmetric import SymmetricBuffer


class FusedGemmContext:
    def __init__(self, ranks=None, group=None, copy_ctas=0):
        self.ranks = list(ranks) if ranks is not None else list(range(process_groups.world_size()))
        self.group = group
        lib = kops._lib()
        lib.kb200_gemm_comm_signal_words.restype = ctypes.c_int
        words = lib.kb200_gemm_comm_signal_words()
        self.signals = SymmetricBuffer(words * 4, group, self.ranks)
        self.signals.tensor(torch.int32).zero_()
        self.rank, self.world = self.signals.rank, self.signals.world
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.gather = [None, None]
        self.stage = [None, None]
        self.epoch = 0
        self._gather_cache = None
        self.copy_ctas = int(copy_ctas)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize()
        self._host_barrier()

    def _host_barrier(self):
        import torch.distributed as dist

        if self.world > 1:
            dist.barrier(group=process_groups.host_group())

    def _ensure(self, slots, parity, nbytes):
        buf = slots[parity]
        if buf is None or buf.nbytes < nbytes:
            # growing is collective: every rank reaches the same call with the same shapes
            torch.cuda.synchronize()
            self._host_barrier()
            if buf is not None:
                buf.close()
            slots[parity] = buf = SymmetricBuffer(int(nbytes), self.group, self.ranks)
        return buf

    def check(self):
        """Raise if a bounded wait inside a fused kernel ran out (reads the status word: synchronises)."""
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise collectives.CommError(f"fused tensor-parallel GEMM gave up waiting for a peer (code 0x{code:x}).")
        kgemm.check_errors()

    def close(self):
        torch.cuda.synchronize()
        for slots in (self.gather, self.stage):
            for i, b in enumerate(slots):
                if b is not None:
                    b.close()
                    slots[i] = None
        self.signals.close()

    def gathered_rows(self, x_rows):
        """All-gather of a row shard for a weight-gradient product.  Projections that read the same activation (query, key
        and value; gate and up) run their backward passes one after the other, so the last result is kept and reused."""
        import torch.distributed as dist

        key = (x_rows.data_ptr(), x_rows._version, tuple(x_rows.shape))
        if self._gather_cache is not None and self._gather_cache[0] == key:
            return self._gather_cache[1]
        full = torch.empty((x_rows.shape[0] * self.world,) + tuple(x_rows.shape[1:]), dtype=x_rows.dtype, device=x_rows.device)
        if self.world > 1:
            dist.all_gather_into_tensor(full, x_rows.contiguous(), group=self.group)
        else:
            full.copy_(x_rows)
        self._gather_cache = (key, full)
        return full

    def drop_cache(self):
        self._gather_cache = None

    # ------------------------------------------------------------------------------------------------
    def all_gather_gemm(self, x_rows, w, b_mn=1, bias=None, act=0, out_dtype=torch.bfloat16):
        """``gather(x_rows) @ w``.  ``x_rows``: [Ms, K] bf16; ``w``: [K, N] (``b_mn=1``) or [N, K] (``b_mn=0``).

        Returns ``(C, gathered)``; ``gathered`` ([world*Ms, K]) is a view of the symmetric buffer, valid until the call
        after next."""
        lib = kops._lib()
        Ms, K = x_rows.shape
        N = w.shape[1] if b_mn else w.shape[0]
        M = Ms * self.world
        self.epoch += 1
        parity = self.epoch & 1
        buf = self._ensure(self.gather, parity, M * K * 2)
        g = buf.tensor(torch.bfloat16)[: M * K].view(M, K)
        g[self.rank * Ms:(self.rank + 1) * Ms].copy_(x_rows)
        out = torch.empty((M, N), dtype=out_dtype, device=x_rows.device)
        err = kgemm._err_flag(x_rows.device)
        code = lib.kb200_gemm_allgather(buf.ptr_array, self.signals.ptr_array, kops._p(w), kops._p(out), kops._p(bias), kops._i(self.rank),
                                        kops._i(self.world), kops._i(Ms), kops._i(N), kops._i(K), kops._ll(w.stride(0)), kops._ll(out.stride(0)),
                                        kops._i(b_mn), kops._i(act), kops._i(1 if out_dtype == torch.float32 else 0), ctypes.c_uint(self.epoch),
                                        kops._i(self.copy_ctas), kops._ll(collectives.comm_timeout_ms()), kops._p(self.status), kops._p(err),
                                        kops._stream())
        kops._check(code, "gemm_allgather")
        return out, g

    def gemm_reduce_scatter(self, a, w, a_mn=0, b_mn=1):
        """Rows ``[rank*Ms, (rank+1)*Ms)`` of ``sum over ranks (a @ w)``.  ``a``: [M, K] (``a_mn=0``) or [K, M] (``a_mn=1``)."""
        lib = kops._lib()
        M = a.shape[1] if a_mn else a.shape[0]
        K = a.shape[0] if a_mn else a.shape[1]
        N = w.shape[1] if b_mn else w.shape[0]
        Ms = M // self.world
        self.epoch += 1
        parity = self.epoch & 1
        buf = self._ensure(self.stage, parity, self.world * Ms * N * 2)
        out = torch.empty((Ms, N), dtype=torch.bfloat16, device=a.device)
        err = kgemm._err_flag(a.device)
        code = lib.kb200_gemm_reduce_scatter(kops._p(a), kops._p(w), buf.ptr_array, self.signals.ptr_array, kops._p(out), kops._i(self.rank),
                                             kops._i(self.world), kops._i(Ms), kops._i(N), kops._i(K), kops._ll(a.stride(0)), kops._ll(w.stride(0)),
                                             kops._i(a_mn), kops._i(b_mn), ctypes.c_uint(self.epoch), kops._ll(collectives.comm_timeout_ms()),
                                             kops._p(self.status), kops._p(err), kops._stream())
        kops._check(code, "gemm_reduce_scatter")
        return out


def supported(rows_per_rank, k, n):
    """Shapes the fused kernels take: 128-row blocks per rank, K and N multiples of 8."""
    return rows_per_rank > 0 and rows_per_rank % 128 == 0 and k % 8 == 0 and n % 8 == 0


class ColumnParallelLinear(torch.autograd.Function):
    """``y[M, N_local] = gather(x_rows) @ w_local``; backward: ``dx_rows = reduce_scatter(dy @ w_localᵀ)``."""

    @staticmethod
    def forward(ctx, x_rows, w, bias, fused):
        b32 = bias.float().contiguous() if bias is not None else None
        y, gathered = fused.all_gather_gemm(x_rows, w, b_mn=1, bias=b32)
        ctx.fused = fused
        ctx.has_bias = bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        # the gathered operand is not kept: backward gathers the shard again (once per distinct input, see gathered_rows)
        ctx.save_for_backward(x_rows, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        x_rows, w = ctx.saved_tensors
        fused = ctx.fused
        xg = fused.gathered_rows(x_rows) if ctx.needs_input_grad[1] else None
        dy = dy if kgemm._ok_2d(dy) else dy.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = fused.gemm_reduce_scatter(dy, w, a_mn=0, b_mn=0)
        if ctx.needs_input_grad[1]:
            K, N = w.shape
            M = dy.shape[0]
            dw = kgemm.gemm(xg, dy, 1, 1, K, N, M, split_k=kgemm.split_k_for(K, N, M, dy.device))
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = kops.column_sum(dy).to(ctx.bias_dtype)
        return dx, dw, db, None


class RowParallelLinear(torch.autograd.Function):
    """``y_rows[Ms, N] = reduce_scatter(x[M, K_local] @ w_local)``; backward: ``dx = gather(dy_rows) @ w_localᵀ``."""

    @staticmethod
    def forward(ctx, x, w, fused):
        ctx.fused = fused
        ctx.save_for_backward(x, w)
        return fused.gemm_reduce_scatter(x, w, a_mn=0, b_mn=1)

    @staticmethod
    def backward(ctx, dy_rows):
        x, w = ctx.saved_tensors
        fused = ctx.fused
        dy_rows = dy_rows if kgemm._ok_2d(dy_rows) else dy_rows.contiguous()
        dx, dyg = fused.all_gather_gemm(dy_rows, w, b_mn=0)
        dw = None
        if ctx.needs_input_grad[1]:
            K, N = w.shape
            M = x.shape[0]
            dw = kgemm.gemm(x, dyg, 1, 1, K, N, M, split_k=kgemm.split_k_for(K, N, M, x.device))
        return (dx if ctx.needs_input_grad[0] else None), dw, None
