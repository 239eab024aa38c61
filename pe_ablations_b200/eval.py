"""Sharded long-context evaluation: batch-sharded perplexity, head-sharded attention.

The eval batch (independent sequences) and the attention heads (independent (batch, head)
problems) partition across the GPUs of one box with no activation exchange.  The only
collective is one all-reduce (SUM) of two scalars per evaluation -- the summed token NLL and
the token count -- issued on the compute stream through ``torch.distributed`` (NCCL over
NVLink on GPUs, gloo on CPU for tests).

The reference evaluates one sequence at a time on one GPU
(scripts/evaluate_ppl_degradation.py:72-111: exp(sum of per-window mean losses weighted by
their token counts / total tokens)); ``perplexity`` computes the same quantity from NLL sums.
"""

from __future__ import annotations

import datetime
import math

import torch
import torch.distributed as dist


def shard_range(n_items: int, world: int, rank: int) -> range:
    """Contiguous, balanced slice of ``n_items`` for ``rank`` (first ``n % world`` ranks get one more)."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world {world}")
    base, extra = divmod(n_items, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def shard_heads(num_heads: int, num_kv_heads: int, world: int, rank: int) -> tuple[range, range]:
    """(query heads, key/value heads) owned by ``rank``: whole GQA groups, so no K/V is shared."""
    if num_kv_heads % world != 0:
        raise ValueError(f"num_kv_heads={num_kv_heads} must be divisible by world={world} to shard by heads")
    g = num_heads // num_kv_heads
    kv = shard_range(num_kv_heads, world, rank)
    return range(kv.start * g, kv.stop * g), kv


REDUCE_TIMEOUT_S = 120.0


def _local_kernel_status(buf: torch.Tensor) -> int:
    """This rank's kernel status code at the host synchronisation the reduction needs anyway."""
    if not buf.is_cuda:
        return 0
    from .ops import poll_device_status

    return poll_device_status(buf.device)


def reduce_loss_sums(nll_sum: torch.Tensor, count: torch.Tensor, group=None,
                     timeout_s: float | None = REDUCE_TIMEOUT_S, status: int | None = None) -> tuple[float, float]:
    """All-reduce (SUM) of the two scalars over ``group``; identity without a process group.

    Two failures are made loud here, at the one place where every rank meets:

    * a kernel of ANY rank that reported an expired wait (its outputs, and so its sums, are
      garbage): each rank adds its status flag (``status``, default: read from this rank's
      device) as a third element, and every rank raises after the reduction if the total is
      non-zero;
    * a rank that is gone (it raised, exited or never joined): the reduction is issued
      asynchronously and waited for at most ``timeout_s`` seconds, after which the survivors
      raise instead of waiting for the process group's default timeout (minutes).
    """
    code = _local_kernel_status(nll_sum) if status is None else int(status)
    buf = torch.stack([nll_sum.double().reshape(()), count.double().reshape(()),
                       torch.tensor(1.0 if code else 0.0, dtype=torch.float64, device=nll_sum.device)])
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        try:
            work = dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group, async_op=True)
            ok = work.wait() if timeout_s is None else work.wait(datetime.timedelta(seconds=float(timeout_s)))
            if ok is False:
                raise RuntimeError("the all-reduce did not complete")
        except Exception as e:     # gloo / NCCL raise their own error types for a lost peer or a timeout
            raise RuntimeError(f"loss-sum reduction failed or timed out after {timeout_s} s: a rank of the "
                               f"evaluation is gone or stuck ({type(e).__name__}: {e})") from e
    nll, cnt, bad = buf.tolist()
    if code or bad != 0.0:
        if code:
            from .ops import check_device_status

            try:
                check_device_status(nll_sum.device)      # clears this rank's word
            except RuntimeError:
                pass
        raise RuntimeError(f"{int(round(bad)) or 1} rank(s) reported expired waits in the attention kernels "
                           f"(this rank's code 0x{code:x}); the reduced sums are invalid")
    return nll, cnt


def perplexity(nll_sum: float, count: float) -> float:
    return math.exp(nll_sum / count) if count > 0 else float("inf")


class GraphedLossSums:
    """``model.loss_sums`` for batches of one fixed shape, captured once into a CUDA graph.

    One 16k-token forward of the 1B shape is about a thousand kernel launches; replayed from a
    graph they run back to back, without the gaps the Python launch path leaves between them.
    Two eager runs on a side stream come first (they perform every first-use host step: kernel
    attributes, TMA descriptor lookups, cuBLAS plans, scratch allocations), then the capture.
    The token ids are copied into a static buffer before each replay; the two result scalars
    are static too and must be consumed (added up) before the next replay.
    """

    @torch.no_grad()
    def __init__(self, model, example_ids: torch.Tensor, autocast_dtype=torch.bfloat16):
        dev = example_ids.device
        self.model, self.autocast_dtype = model, autocast_dtype
        self.static_ids = example_ids.clone()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                self._run()
        torch.cuda.current_stream(dev).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.nll, self.cnt = self._run()

    def _run(self):
        if self.autocast_dtype is not None:
            with torch.autocast("cuda", dtype=self.autocast_dtype):
                return self.model.loss_sums(self.static_ids)
        return self.model.loss_sums(self.static_ids)

    def __call__(self, ids: torch.Tensor):
        if ids.shape != self.static_ids.shape:
            raise ValueError(f"captured for token ids of shape {tuple(self.static_ids.shape)}, got {tuple(ids.shape)}")
        self.static_ids.copy_(ids)
        self.graph.replay()
        return self.nll, self.cnt


@torch.no_grad()
def evaluate_shard(model, input_ids: torch.Tensor, micro_batch: int = 1, autocast_dtype=torch.bfloat16,
                   graphed: GraphedLossSums | None = None):
    """NLL sum and token count of this rank's sequences [n, S] (device tensors).  With ``graphed``
    (captured for ``micro_batch`` sequences of this length) full micro-batches replay the graph."""
    dev = input_ids.device
    nll = torch.zeros((), dtype=torch.float64, device=dev)
    cnt = torch.zeros((), dtype=torch.float64, device=dev)
    for i in range(0, input_ids.shape[0], micro_batch):
        ids = input_ids[i:i + micro_batch]
        if graphed is not None and ids.shape == graphed.static_ids.shape:
            a, c = graphed(ids)
        elif autocast_dtype is not None and dev.type == "cuda":
            with torch.autocast("cuda", dtype=autocast_dtype):
                a, c = model.loss_sums(ids)
        else:
            a, c = model.loss_sums(ids)
        nll += a.double()
        cnt += c.double()
    return nll, cnt


@torch.no_grad()
def sharded_perplexity(model, all_input_ids: torch.Tensor, rank: int, world: int, micro_batch: int = 1,
                       autocast_dtype=torch.bfloat16, group=None, graphed: GraphedLossSums | None = None,
                       timeout_s: float | None = REDUCE_TIMEOUT_S) -> dict:
    """Perplexity of ``all_input_ids`` [N, S] with sequences sharded over ``world`` ranks.  Raises on
    every rank if any rank's kernels reported an expired wait, or if a rank does not arrive at
    the reduction within ``timeout_s`` seconds (see ``reduce_loss_sums``)."""
    mine = shard_range(all_input_ids.shape[0], world, rank)
    ids = all_input_ids[mine.start:mine.stop].to(next(model.parameters()).device, non_blocking=True)
    nll, cnt = evaluate_shard(model, ids, micro_batch, autocast_dtype, graphed)
    tot_nll, tot_cnt = reduce_loss_sums(nll, cnt, group, timeout_s)
    return {"nll_sum": tot_nll, "count": tot_cnt, "loss": tot_nll / max(tot_cnt, 1.0),
            "perplexity": perplexity(tot_nll, tot_cnt), "local_sequences": len(mine)}


# ---- the 1B-shape 16k-context evaluation of the benchmark configuration list -----------------
MODEL_1B = dict(vocab_size=32000, hidden_dim=2048, num_layers=16, num_heads=16, num_kv_heads=16, head_dim=128,
                ffn_dim=5632, max_seq_len=16384, pe_mode="fpope", fpope_d_rope=64, fpope_num_fourier_terms=16,
                fpope_sigma=0.3, fpope_training_length=16384, fpope_delta_init="uniform")


def cast_matmul_weights(model, dtype=torch.bfloat16):
    """Store the weights of every Linear / Embedding in ``dtype`` (norm weights and positional
    parameters stay fp32), so that a bf16-autocast forward does not re-cast them per call."""
    import torch.nn as nn

    seen = set()
    for m in model.modules():
        if isinstance(m, (nn.Linear, nn.Embedding)) and id(m.weight) not in seen:
            seen.add(id(m.weight))
            m.weight.data = m.weight.data.to(dtype)
    return model


def build_1b_model(device, seed: int = 0, dtype=torch.bfloat16):
    """Random-init (N(0, 0.02^2), seeded) 1B-shape FoPE+PoPE decoder on ``device``."""
    from .model import Transformer, TransformerConfig

    torch.manual_seed(seed)
    with torch.device(device):
        model = Transformer(TransformerConfig(**MODEL_1B)).eval()
    return cast_matmul_weights(model, dtype) if dtype is not None else model
