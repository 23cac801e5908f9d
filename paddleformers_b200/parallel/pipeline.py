"""Pipeline parallelism: stage partitioning, schedules (FThenB, 1F1B, interleaved 1F1B, zero-bubble, and the V placement
with split backward) and the execution engine.

Roles of the reference's ``GeneralModelForCausalLMPipe`` (paddleformers/nn/pp_model.py:509-688: layer descriptions,
``seg_method``, empty layers, virtual stages, shared embeddings) and of Fleet's ``forward_backward_pipeline`` driven by
the trainer (paddleformers/trainer/trainer.py:4531-4580). Point-to-point traffic stays on NCCL send/recv, as two
independent communicators (one per direction of dataflow: activations forward, gradients backward) so that messages
of different kinds between the same pair of ranks can never be matched against each other, and on their own CUDA
streams so that transfers overlap compute.

The schedules are generated as plain lists of actions per stage; ``simulate`` checks any schedule for dependency
order and reports the peak number of in-flight micro-batches per stage, which the CPU tests assert.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import functional as F
from ..transformers.model_utils import PretrainedModel
from .topology import ParallelState, get_parallel_state


# ---------------------------------------------------------------------------------------------------------------
# partitioning
# ---------------------------------------------------------------------------------------------------------------
V_SCHEDULES = ("zbv", "zb-v", "zb_v", "dualpipev", "dual_pipe_v")


def is_v_schedule(name: Optional[str]) -> bool:
    return str(name or "").lower() in V_SCHEDULES


def virtual_stage(stage: int, chunk: int, P: int, v_shape: bool = False) -> int:
    """Position of (stage, chunk) in the model's layer order. Interleaved placement walks the stages once per chunk
    (chunk * P + stage); the V placement walks them down with chunk 0 and back up with chunk 1, so that the first and the
    last part of the model share stage 0 and the turn at the last stage needs no communication."""
    if v_shape:
        return stage if chunk == 0 else 2 * P - 1 - stage
    return chunk * P + stage


def stage_of_virtual(vs: int, P: int, v_shape: bool = False) -> Tuple[int, int]:
    """Inverse of ``virtual_stage``: (stage, chunk)."""
    if v_shape:
        return (vs, 0) if vs < P else (2 * P - 1 - vs, 1)
    return vs % P, vs // P


def partition_layers(num_layers: int, num_stages: int, num_virtual: int = 1, empty_head: int = 0, empty_tail: int = 0,
                     weights: Optional[Sequence[float]] = None, v_shape: bool = False) -> List[List[range]]:
    """Split ``num_layers`` decoder layers over ``num_stages * num_virtual`` virtual stages.

    Returns ``parts[stage][chunk] = range of layer ids``. Empty layers count as layers of zero cost placed before the
    first / after the last decoder layer (``num_empty_layers_add_in_head/tail``) which shifts real layers away from
    the stages that also hold the embedding / head. ``weights`` gives a per-layer cost for non-uniform splits."""
    n_virtual = num_stages * num_virtual
    total = num_layers + empty_head + empty_tail
    if weights is None:
        base, rem = divmod(total, n_virtual)
        sizes = [base + (1 if i < rem else 0) for i in range(n_virtual)]
    else:
        assert len(weights) == total
        # greedy prefix split: close a virtual stage once its cost reaches the running average of what is left
        sizes, start = [], 0
        remaining_cost = float(sum(weights))
        for v in range(n_virtual):
            slots_left = n_virtual - v
            if slots_left == 1:
                sizes.append(total - start)
                break
            target = remaining_cost / slots_left
            acc, cnt = 0.0, 0
            while start + cnt < total - (slots_left - 1) and (cnt == 0 or acc + weights[start + cnt] / 2 <= target):
                acc += weights[start + cnt]
                cnt += 1
            sizes.append(cnt)
            start += cnt
            remaining_cost -= acc
    bounds, pos = [], 0
    for s in sizes:
        bounds.append((pos, pos + s))
        pos += s
    parts: List[List[range]] = [[None] * num_virtual for _ in range(num_stages)]
    for v, (lo, hi) in enumerate(bounds):
        stage, chunk = stage_of_virtual(v, num_stages, v_shape)
        real_lo = min(max(lo - empty_head, 0), num_layers)
        real_hi = min(max(hi - empty_head, 0), num_layers)
        parts[stage][chunk] = range(real_lo, real_hi)
    return parts


# ---------------------------------------------------------------------------------------------------------------
# schedules
# ---------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class Action:
    kind: str    # "F" or "B"
    chunk: int   # virtual chunk on this stage
    mb: int      # micro-batch id


def schedule_fthenb(stage: int, P: int, M: int, V: int = 1) -> List[Action]:
    acts = [Action("F", c, m) for c in range(V) for m in range(M)]
    acts += [Action("B", c, m) for c in reversed(range(V)) for m in range(M)]
    return acts


def schedule_1f1b(stage: int, P: int, M: int) -> List[Action]:
    warm = min(P - stage - 1, M)
    acts = [Action("F", 0, m) for m in range(warm)]
    f, b = warm, 0
    while f < M:
        acts.append(Action("F", 0, f)); f += 1
        acts.append(Action("B", 0, b)); b += 1
    while b < M:
        acts.append(Action("B", 0, b)); b += 1
    return acts


def schedule_interleaved(stage: int, P: int, M: int, V: int) -> List[Action]:
    """Interleaved 1F1B (virtual pipeline): micro-batches advance in groups of P through the V chunks."""
    assert M % P == 0, "interleaved schedule needs the number of micro-batches to be a multiple of the pipeline degree"
    total = M * V

    def fwd_ids(k):
        group, within = divmod(k, P * V)
        chunk = within // P
        return chunk, group * P + within % P

    def bwd_ids(k):
        chunk, mb = fwd_ids(k)
        return V - 1 - chunk, mb

    warm = min((P - stage - 1) * 2 + (V - 1) * P, total)
    acts = [Action("F", *fwd_ids(k)) for k in range(warm)]
    f, b = warm, 0
    while f < total:
        acts.append(Action("F", *fwd_ids(f))); f += 1
        acts.append(Action("B", *bwd_ids(b))); b += 1
    while b < total:
        acts.append(Action("B", *bwd_ids(b))); b += 1
    return acts


def schedule_zero_bubble(stage: int, P: int, M: int) -> List[Action]:
    """1F1B with the backward pass split into B (gradient w.r.t. the stage input: the part the previous stage waits
    for) and W (weight gradients, needed only before the optimizer step), W running right after its B. The chain of
    backward dependencies between stages then advances in B-sized instead of (B + W)-sized hops, which removes the W
    share of the warm-up and cool-down bubbles: with unit costs the makespan falls from 3M + 3(P - 1) to
    3M + 2(P - 1) at 1F1B's activation memory (checked by ``simulate`` in the tests). The reference attacks the same
    bubble with its DualPipeV / overlapped schedule nodes
    (paddleformers/cli/train/deepseek_v3_pretrain/modeling_pp.py:535-606)."""
    warm = min(P - stage - 1, M)
    acts = [Action("F", 0, m) for m in range(warm)]
    f = warm
    for b in range(M):
        if f < M:
            acts.append(Action("F", 0, f)); f += 1
        acts.append(Action("B", 0, b))
        acts.append(Action("W", 0, b))
    return acts


def schedule_zbv(stage: int, P: int, M: int) -> List[Action]:
    """Schedule for the V placement (two chunks per stage, chunk 0 running down the stages and chunk 1 back up) with the
    backward pass split into B and W: the family the reference reaches through ``use_dualpipev`` and its overlapped schedule
    nodes (paddleformers/trainer/training_args.py:2073-2087, paddleformers/cli/train/deepseek_v3_pretrain/modeling_pp.py:
    535-606). Built by list scheduling on unit costs: every stage runs, at each step, the first ready action in the priority
    order B (which the neighbour waits for), then forward of chunk 1, forward of chunk 0, and W only when nothing else is
    ready; forwards of chunk 0 are admitted while fewer than P + 1 micro-batch chunks are alive on the stage, which keeps every
    stage at about 2P half-size chunks: the activation memory of 1F1B's first stage, but the same on all stages. (A larger
    cap trades memory for a smaller bubble; ``_zbv_all`` takes it as a parameter.) The loss and the embedding sit on the same
    stage, so the backward of a micro-batch can start right after its forward returns to stage 0."""
    return _zbv_all(P, M)[stage]


def ZBV_LIVE_CAP(P: int) -> int:
    """Chunk-0 forwards are admitted while fewer than this many chunks are alive on a stage."""
    return P + 1


_ZBV_CACHE: Dict[Tuple[int, int, int], List[List[Action]]] = {}


def _zbv_all(P: int, M: int, max_live: Optional[int] = None) -> List[List[Action]]:
    cap = int(max_live) if max_live else ZBV_LIVE_CAP(P)
    if (P, M, cap) in _ZBV_CACHE:
        return _ZBV_CACHE[(P, M, cap)]
    last = 2 * P - 1
    done_f: Dict[Tuple[int, int], int] = {}       # (virtual stage, micro-batch) -> finish time
    done_b: Dict[Tuple[int, int], int] = {}
    out: List[List[Action]] = [[] for _ in range(P)]
    nf = [[0, 0] for _ in range(P)]                # next micro-batch to run forward, per chunk
    nb = [[0, 0] for _ in range(P)]
    wq: List[List[Tuple[int, int]]] = [[] for _ in range(P)]
    live = [0] * P
    t, total, emitted = 0, P * M * 2 * 3, 0
    while emitted < total:
        step = []
        for s in range(P):
            choice = None
            # B: chunk 1 first (it is earlier in the backward order)
            for c in (1, 0):
                m = nb[s][c]
                if m >= M:
                    continue
                vs = virtual_stage(s, c, P, True)
                ready = done_f.get((vs, m), 1 << 30) <= t and (vs == last or done_b.get((vs + 1, m), 1 << 30) <= t)
                if ready:
                    choice = ("B", c, m)
                    break
            if choice is None:
                for c in (1, 0):
                    m = nf[s][c]
                    if m >= M:
                        continue
                    vs = virtual_stage(s, c, P, True)
                    if vs > 0 and done_f.get((vs - 1, m), 1 << 30) > t:
                        continue
                    if c == 0 and live[s] >= cap:
                        continue
                    choice = ("F", c, m)
                    break
            if choice is None and wq[s]:
                c, m = wq[s][0]
                choice = ("W", c, m)
            if choice is not None:
                step.append((s, choice))
        if not step and emitted < total:
            t += 1
            if t > 16 * (total + P):
                raise RuntimeError("zbv schedule construction did not terminate")
            continue
        for s, (kind, c, m) in step:
            vs = virtual_stage(s, c, P, True)
            out[s].append(Action(kind, c, m))
            emitted += 1
            if kind == "F":
                done_f[(vs, m)] = t + 1
                nf[s][c] += 1
                live[s] += 1
            elif kind == "B":
                done_b[(vs, m)] = t + 1
                nb[s][c] += 1
                wq[s].append((c, m))
            else:
                wq[s].pop(0)
                live[s] -= 1
        t += 1
    _ZBV_CACHE[(P, M, cap)] = out
    return out


def make_schedule(name: str, stage: int, P: int, M: int, V: int = 1) -> List[Action]:
    name = name.lower()
    if name in V_SCHEDULES:
        assert V == 2, "the V placement has exactly two chunks per stage"
        return schedule_zbv(stage, P, M)
    if name in ("fthenb", "f-then-b"):
        return schedule_fthenb(stage, P, M, V)
    if name in ("zb", "zbh1", "zero_bubble", "zero-bubble"):
        assert V == 1, "the zero-bubble schedule is defined for one chunk per stage"
        return schedule_zero_bubble(stage, P, M)
    if V > 1 or name in ("interleaved", "vpp"):
        return schedule_interleaved(stage, P, M, max(V, 1))
    return schedule_1f1b(stage, P, M)


def simulate(schedules: List[List[Action]], P: int, V: int, cost: Optional[Dict[str, float]] = None,
             v_shape: bool = False) -> Dict[str, object]:
    """Runs all stages' action lists as a timed simulation: every stage executes its list in order, an action starts
    when the stage is free and its dependencies have finished. ``cost`` maps action kinds to durations; by default a
    forward costs 1, a fused backward 2, and in schedules that split it B and W cost 1 each. Raises on deadlock;
    returns makespan, bubble fraction (idle share of the busiest stage's timeline) and peak live activations."""
    split = any(a.kind == "W" for sch in schedules for a in sch)
    cost = cost or ({"F": 1.0, "B": 1.0, "W": 1.0} if split else {"F": 1.0, "B": 2.0})
    fin_f: Dict[Tuple[int, int], float] = {}
    fin_b: Dict[Tuple[int, int], float] = {}
    pos = [0] * P
    free = [0.0] * P
    live = [0] * P
    peak = [0] * P
    n_actions = sum(len(s) for s in schedules)
    finished = 0
    last_virtual = P * V - 1
    while finished < n_actions:
        progressed = False
        for s in range(P):
            while pos[s] < len(schedules[s]):
                a = schedules[s][pos[s]]
                vs = virtual_stage(s, a.chunk, P, v_shape)
                if a.kind == "F":
                    deps = [] if vs == 0 else [fin_f.get((vs - 1, a.mb))]
                elif a.kind == "B":
                    deps = [fin_f.get((vs, a.mb))] + ([] if vs == last_virtual else [fin_b.get((vs + 1, a.mb))])
                else:
                    deps = [fin_b.get((vs, a.mb))]
                if any(d is None for d in deps):
                    break
                start = max([free[s]] + deps)
                end = start + cost[a.kind]
                free[s] = end
                if a.kind == "F":
                    fin_f[(vs, a.mb)] = end
                    live[s] += 1
                    peak[s] = max(peak[s], live[s])
                elif a.kind == "B":
                    fin_b[(vs, a.mb)] = end
                    if not split:
                        live[s] -= 1
                else:
                    live[s] -= 1
                pos[s] += 1
                finished += 1
                progressed = True
        if not progressed:
            raise RuntimeError(f"pipeline schedule deadlocks at positions {pos}")
    makespan = max(free)
    work = max(sum(cost[a.kind] for a in sch) for sch in schedules)
    return {"makespan": makespan, "bubble_fraction": 1.0 - work / makespan, "peak_live": peak}


# ---------------------------------------------------------------------------------------------------------------
# stage model
# ---------------------------------------------------------------------------------------------------------------
class PipelineStageModel(PretrainedModel):
    """The chunks of a decoder that live on this pipeline stage. Chunk c of stage s is virtual stage c * P + s.
    The embedding lives on virtual stage 0, the final norm, MTP layers and head on the last one; with tied
    embeddings both ends hold a copy whose gradients are summed over the two owners after the backward pass
    (the reference's SharedLayerDesc, paddleformers/nn/pp_model.py:582-594)."""

    def __init__(self, config, dtype=None, device=None, ps: Optional[ParallelState] = None):
        super().__init__(config)
        from ..models.modeling import DecoderModel, MTPLayer, RMSNorm, _resolve_dtype

        ps = ps or get_parallel_state()
        self.config = config
        self.ps = ps
        P, V = ps.degrees.pp, max(int(getattr(config, "virtual_pipeline_model_parallel_size", 1) or 1), 1)
        # V placement (schedule "zbv"): two chunks per stage, the model runs down the stages and back up, so that stage 0
        # holds both the embedding and the head
        self.v_shape = is_v_schedule(getattr(config, "pipeline_schedule", None)) and P > 1
        if self.v_shape:
            V = 2
        self.P, self.V, self.stage = P, V, ps.coord["pp"]
        dtype = dtype if dtype is not None else _resolve_dtype(config.dtype)
        parts = partition_layers(config.num_hidden_layers, P, V, int(getattr(config, "num_empty_layers_add_in_head", 0) or 0),
                                 int(getattr(config, "num_empty_layers_add_in_tail", 0) or 0), v_shape=self.v_shape)
        self.layer_ranges = parts[self.stage]
        self.chunks = nn.ModuleList()
        last_stage = 0 if self.v_shape else P - 1
        for c, rng in enumerate(self.layer_ranges):
            first = self.stage == 0 and c == 0
            last = self.stage == last_stage and c == V - 1
            # with the V placement a tied / MTP embedding on the last chunk is the first chunk's own parameter (set below)
            self.chunks.append(DecoderModel(config, dtype=dtype, device=device, layer_range=rng,
                                            with_embedding=first or (last and config.tie_word_embeddings and not self.v_shape),
                                            with_final_norm=last))
        self.is_first = self.stage == 0
        self.is_last = self.stage == last_stage
        if self.v_shape and self.is_last and (config.tie_word_embeddings or int(getattr(config, "num_nextn_predict_layers", 0) or 0)):
            self.chunks[-1].embed_tokens = self.chunks[0].embed_tokens       # one parameter, two users: autograd sums the gradients
        self.lm_head = None
        self.mtp_layers = nn.ModuleList()
        if self.is_last:
            if not config.tie_word_embeddings:
                self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False, dtype=dtype, device=device)
            n_mtp = int(getattr(config, "num_nextn_predict_layers", 0) or 0)
            self.mtp_layers = nn.ModuleList([MTPLayer(config, config.num_hidden_layers + i, dtype=dtype, device=device) for i in range(n_mtp)])
            if n_mtp and self.chunks[-1].embed_tokens is None and not self.v_shape:
                # MTP needs token embeddings on the last stage: a tied copy of the input embedding, of the same kind (a
                # vocabulary shard under tensor parallelism) so that the two stages can sum their gradients
                if ps.degrees.mp > 1:
                    from .tensor_parallel import VocabParallelEmbedding

                    self.chunks[-1].embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size, False,
                                                                          dtype=dtype, device=device)
                else:
                    self.chunks[-1].embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, dtype=dtype, device=device)
                self.chunks[-1].embed_tokens.weight.pp_shared = "embed_tokens"
        if not self.v_shape:
            if self.is_first and self.chunks[0].embed_tokens is not None and (config.tie_word_embeddings or getattr(config, "num_nextn_predict_layers", 0)):
                self.chunks[0].embed_tokens.weight.pp_shared = "embed_tokens"
            if self.is_last and config.tie_word_embeddings and self.chunks[-1].embed_tokens is not None:
                self.chunks[-1].embed_tokens.weight.pp_shared = "embed_tokens"
        self.loss_accumulation_steps = 1
        self.ignore_index = -100
        std = config.initializer_range
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, 0.0, std)
        from ..nn.moe import GroupedExperts, TopkRouter

        for m in self.modules():
            if isinstance(m, GroupedExperts):
                nn.init.normal_(m.gate_up_proj, 0.0, std); nn.init.normal_(m.down_proj, 0.0, std)
            elif isinstance(m, TopkRouter):
                nn.init.normal_(m.weight, 0.0, std)

    def head_weight(self):
        return self.lm_head.weight if self.lm_head is not None else self.chunks[-1].embed_tokens.weight

    # ---- names of this stage's parameters in the un-partitioned model (checkpoints use those)
    def global_param_name(self, local_name: str) -> str:
        if local_name.startswith("chunks."):
            rest = local_name.split(".", 2)[2]
            return "model." + rest
        return local_name  # lm_head.*, mtp_layers.*

    def owns_global_param(self, local_name: str) -> bool:
        # the input embedding belongs to the first stage; the copy on the last stage (tied head / MTP) is not saved
        if ".embed_tokens." in local_name and not self.is_first:
            return False
        return True

    def weight_map(self):
        from ..models.modeling import build_weight_map

        return build_weight_map(self.config)

    def _init_weights(self, module):
        pass

    def forward_chunk(self, c: int, x, batch, ctx):
        model = self.chunks[c]
        if self.is_first and c == 0:
            x = model.embed(batch["input_ids"])
        hidden, residual = model.run_layers(x, None, ctx)
        last = self.is_last and c == self.V - 1
        if last:
            if model.norm is not None:
                hidden = model.norm(hidden, residual)[0] if residual is not None else model.norm(hidden)
            return hidden
        return hidden + residual if residual is not None else hidden

    def _head_loss(self, hidden, labels, scale, gather: bool = False):
        """Head + cross entropy on this stage: under sequence parallelism the token slices are gathered first (every rank then
        holds all rows; the backward pass keeps this rank's slice); a head that is a vocabulary shard (tied to a
        vocabulary-parallel embedding) goes through the vocabulary-parallel loss."""
        ps = get_parallel_state()
        tp, w = ps.degrees.mp, self.head_weight()
        if gather and tp > 1 and getattr(self.chunks[-1], "sp", False):
            from .tensor_parallel import GatherOp

            hidden = GatherOp.apply(hidden, ps.group("mp"))
        if tp > 1 and w.shape[0] != self.config.vocab_size:
            from .vocab_parallel_loss import vocab_parallel_linear_cross_entropy

            return vocab_parallel_linear_cross_entropy(hidden, w, labels, self.ignore_index, scale)[0]
        return F.fused_linear_cross_entropy(hidden, w, labels, self.ignore_index, 2048, scale)[0]

    def loss(self, hidden, batch, ctx):
        from ..models.modeling import label_norm

        labels = batch["labels"].reshape(-1)
        count = (labels != self.ignore_index).sum()
        # ranks of a context / segment parallel group divide by the labelled tokens of the whole sequence
        scale = 1.0 / (label_norm(count) * float(self.loss_accumulation_steps))
        loss = self._head_loss(hidden, labels, scale, gather=True)
        if len(self.mtp_layers) > 0:
            ps = get_parallel_state()
            if getattr(self.chunks[-1], "sp", False) or ps.degrees.cp > 1 or ps.degrees.sep > 1:
                raise NotImplementedError("multi-token-prediction layers on a pipeline stage are implemented without sequence, "
                                          "context and segment parallelism")
            ids, lab, h = batch["input_ids"], batch["labels"], hidden
            # the weight of the term goes into the scale of the fused head + loss (its weight gradient is written during the
            # forward pass and would not see a factor applied afterwards)
            w = float(getattr(self.config, "mtp_loss_scaling_factor", 0.1)) / len(self.mtp_layers)
            extra = []
            for layer in self.mtp_layers:
                ids = torch.cat([ids[:, 1:], ids[:, -1:]], 1)
                lab = torch.cat([lab[:, 1:], torch.full_like(lab[:, -1:], self.ignore_index)], 1)
                table = self.chunks[-1].embed_tokens
                emb = table(ids) if ps.degrees.mp > 1 else F.embedding(ids, table.weight)
                h = layer(h, emb.reshape(-1, self.config.hidden_size), ctx)
                flat = lab.reshape(-1)
                cnt = (flat != self.ignore_index).sum()
                sc = w / (cnt.clamp(min=1).float() * float(self.loss_accumulation_steps))
                extra.append(self._head_loss(h, flat, sc))
            loss = loss + torch.stack(extra).sum()
        return loss


def build_pipeline_model(config, dtype=None, device=None, **kw):
    return PipelineStageModel(config, dtype=dtype, device=device)


# ---------------------------------------------------------------------------------------------------------------
# engine
# ---------------------------------------------------------------------------------------------------------------
class PipelineEngine:
    """Executes one optimizer step worth of micro-batches with the chosen schedule."""

    def __init__(self, model: PipelineStageModel, ps: Optional[ParallelState] = None, schedule: str = "1F1B",
                 num_virtual_stages: int = 1):
        self.model = model
        self.ps = ps or get_parallel_state()
        self.P, self.V = self.ps.degrees.pp, model.V
        self.stage = self.ps.coord["pp"]
        self.schedule_name = schedule
        ranks = self.ps.group_ranks["pp"]
        self.ranks = ranks
        self.v_shape = bool(getattr(model, "v_shape", False))
        if is_v_schedule(schedule) != self.v_shape and self.P > 1:
            raise ValueError(f"schedule {schedule!r} and the model's chunk placement disagree: build the model with the same "
                             "pipeline_schedule in its configuration")
        self.prev_rank = ranks[(self.stage - 1) % self.P]
        self.next_rank = ranks[(self.stage + 1) % self.P]
        # two communicators: activations travel on one, gradients on the other
        self.fwd_group, self.bwd_group, self._shared_group = _pp_comm_groups(self.ps)

    # -- communication helpers (blocking semantics on the consumer side; producers are asynchronous)
    def _send(self, t, dst, group, pending):
        pending.append(dist.isend(t.contiguous(), dst=dst, group=group))

    def _recv(self, shape, dtype, device, src, group):
        buf = torch.empty(shape, dtype=dtype, device=device)
        dist.recv(buf, src=src, group=group)
        return buf

    def _owner(self, vs: int) -> int:
        """Stage that holds virtual stage ``vs``."""
        return stage_of_virtual(vs, self.P, self.v_shape)[0]

    def forward_backward(self, micro_batches: List[Dict[str, torch.Tensor]]) -> torch.Tensor:
        model, P, V, s = self.model, self.P, self.V, self.stage
        M = len(micro_batches)
        model.loss_accumulation_steps = M
        acts = make_schedule(self.schedule_name, s, P, M, V)
        H = model.config.hidden_size
        dev = next(model.parameters()).device
        dtype = next((p.dtype for n, p in model.named_parameters() if "gate.weight" not in n), torch.float32)
        saved: Dict[Tuple[int, int], Tuple[Optional[torch.Tensor], torch.Tensor]] = {}
        ctxs: Dict[int, object] = {}
        pending: List[object] = []
        total_loss = torch.zeros((), dtype=torch.float32, device=dev)
        last_virtual = P * V - 1
        split_w = any(a.kind == "W" for a in acts)
        local_fwd: Dict[Tuple[int, int], torch.Tensor] = {}     # hand-over between two chunks of this stage (V placement)
        local_bwd: Dict[Tuple[int, int], torch.Tensor] = {}
        # expert-parallel exchange buffers are kept per micro-batch in flight (forward done, backward pending)
        from .fused_ep import SlotAllocator, set_micro_batch_slot

        slots = SlotAllocator(chunks_per_micro_batch=V)
        for a in acts:
            if a.kind == "W":
                F.WeightGradStore.run_group()      # the weight-gradient GEMMs queued by the matching B
                continue
            vs = virtual_stage(s, a.chunk, P, self.v_shape)
            batch = micro_batches[a.mb]
            B, S = batch["input_ids"].shape
            if a.mb not in ctxs:
                kend = batch.get("attn_mask_startend_row_indices", batch.get("kend"))
                kend_full = batch.get("full_attn_mask_startend_row_indices")
                ctxs[a.mb] = model.chunks[0].make_context(batch["input_ids"], batch.get("position_ids"),
                                                          kend.reshape(B, -1) if kend is not None else None,
                                                          batch.get("cp_global_positions"), batch.get("cp_full_seq_len"),
                                                          kend_full.reshape(B, -1) if kend_full is not None else None)
            ctx = ctxs[a.mb]
            # neighbours in the model's layer order; with the V placement the turn at the last stage stays on this rank
            src_stage = self._owner(vs - 1) if vs > 0 else None
            dst_stage = self._owner(vs + 1) if vs < last_virtual else None
            set_micro_batch_slot(slots.acquire(a.mb))
            if a.kind == "F":
                x_in = None
                if vs > 0:
                    if src_stage == s:
                        x_in = local_fwd.pop((vs - 1, a.mb))
                    else:
                        # under sequence parallelism a stage hands over this rank's slice of the tokens
                        rows = B * S // self.ps.degrees.mp if getattr(model.chunks[0], "sp", False) else B * S
                        x_in = self._recv((rows, H), dtype, dev, self.ranks[src_stage], self.fwd_group)
                    x_in.requires_grad_(True)
                out = model.forward_chunk(a.chunk, x_in, batch, ctx)
                if vs == last_virtual:
                    loss = model.loss(out, batch, ctx)
                    total_loss += loss.detach()
                    saved[(a.chunk, a.mb)] = (x_in, loss)
                else:
                    if dst_stage == s:
                        local_fwd[(vs, a.mb)] = out.detach()
                    else:
                        self._send(out.detach(), self.ranks[dst_stage], self.fwd_group, pending)
                    saved[(a.chunk, a.mb)] = (x_in, out)
            else:
                x_in, out = saved.pop((a.chunk, a.mb))
                if split_w:
                    F.WeightGradStore.begin_group()
                try:
                    if vs == last_virtual:
                        out.backward()
                    else:
                        if dst_stage == s:
                            g = local_bwd.pop((vs + 1, a.mb))
                        else:
                            g = self._recv(tuple(out.shape), out.dtype, dev, self.ranks[dst_stage], self.bwd_group)
                        torch.autograd.backward(out, g)
                finally:
                    if split_w:
                        F.WeightGradStore.end_group()
                slots.backward_done(a.mb)
                if vs > 0:
                    if src_stage == s:
                        local_bwd[(vs, a.mb)] = x_in.grad
                    else:
                        self._send(x_in.grad, self.ranks[src_stage], self.bwd_group, pending)
        F.WeightGradStore.run_all()
        set_micro_batch_slot(0)
        for w in pending:
            w.wait()
        self._sync_shared_embeddings()
        # every stage reports the same loss: the last stage owns it
        if P > 1:
            src = self.ps.group_ranks["pp"][self._owner(last_virtual)]
            dist.broadcast(total_loss, src=src, group=self.ps.group("pp"))
        return total_loss

    @torch.no_grad()
    def forward_only(self, micro_batches: List[Dict[str, torch.Tensor]]):
        """Evaluation: every micro-batch runs down the virtual stages in order, nothing is kept for a backward pass. Returns
        (sum over micro-batches of mean loss x labelled tokens, labelled tokens), the same on every stage."""
        model, P, V, s = self.model, self.P, self.V, self.stage
        H = model.config.hidden_size
        dev = next(model.parameters()).device
        dtype = next((p.dtype for n, p in model.named_parameters() if "gate.weight" not in n), torch.float32)
        last_virtual = P * V - 1
        saved_accum, model.loss_accumulation_steps = model.loss_accumulation_steps, 1
        both = torch.zeros(2, dtype=torch.float64, device=dev)
        mine = sorted((virtual_stage(s, c, P, self.v_shape), c) for c in range(V))
        try:
            for batch in micro_batches:
                B, S = batch["input_ids"].shape
                kend = batch.get("attn_mask_startend_row_indices", batch.get("kend"))
                kend_full = batch.get("full_attn_mask_startend_row_indices")
                ctx = model.chunks[0].make_context(batch["input_ids"], batch.get("position_ids"),
                                                   kend.reshape(B, -1) if kend is not None else None,
                                                   batch.get("cp_global_positions"), batch.get("cp_full_seq_len"),
                                                   kend_full.reshape(B, -1) if kend_full is not None else None)
                handed = None
                for vs, c in mine:
                    x_in = None
                    if vs > 0:
                        if self._owner(vs - 1) == s:
                            x_in = handed
                        else:
                            rows = B * S // self.ps.degrees.mp if getattr(model.chunks[0], "sp", False) else B * S
                            x_in = self._recv((rows, H), dtype, dev, self.ranks[self._owner(vs - 1)], self.fwd_group)
                    out = model.forward_chunk(c, x_in, batch, ctx)
                    if vs == last_virtual:
                        pair = torch.stack([model.loss(out, batch, ctx).double(), (batch["labels"] != model.ignore_index).sum().double()])
                        for axis in ("cp", "sep"):      # slices of one sequence: the mean of their losses, the sum of their counts
                            if getattr(self.ps.degrees, axis) > 1:
                                dist.all_reduce(pair, group=self.ps.group(axis))
                                pair[0] /= getattr(self.ps.degrees, axis)
                        both += torch.stack([pair[0] * pair[1], pair[1]])
                    elif self._owner(vs + 1) == s:
                        handed = out
                    else:
                        pending: List[object] = []
                        self._send(out, self.ranks[self._owner(vs + 1)], self.fwd_group, pending)
                        for w in pending:
                            w.wait()
        finally:
            model.loss_accumulation_steps = saved_accum
        if P > 1:
            dist.broadcast(both, src=self.ps.group_ranks["pp"][self._owner(last_virtual)], group=self.ps.group("pp"))
        return both[0], both[1]

    def _sync_shared_embeddings(self):
        """Sum the gradients of parameters that exist on both the first and the last stage (tied embeddings, MTP
        embedding copy)."""
        shared = [p for p in self.model.parameters() if getattr(p, "pp_shared", None)]
        if not shared or self.P == 1 or self.v_shape:
            return
        if not (self.model.is_first or self.model.is_last):
            return
        for p in shared:
            g = getattr(p, "main_grad", None)
            if g is not None and p.grad is not None:
                g.add_(p.grad.to(g.dtype))          # what autograd left in .grad belongs to the sum as well
                p.grad = None
            if g is None:
                g = p.grad
            if g is not None:
                dist.all_reduce(g, group=self._shared_group)


_PP_GROUPS = {}


def _pp_comm_groups(ps: ParallelState):
    """(forward communicator, backward communicator, first+last stage group) of this rank's pipeline group. Creating
    groups is collective over the whole job, so every rank builds every pipeline group's communicators."""
    key = id(ps)
    if key not in _PP_GROUPS:
        fwd = bwd = shared = None
        if ps.degrees.pp > 1 and dist.is_initialized():
            for ranks in ps.topo.comm_list("pp"):
                f = dist.new_group(ranks=ranks)
                b = dist.new_group(ranks=ranks)
                sh = dist.new_group(ranks=[ranks[0], ranks[-1]])
                if ps.global_rank in ranks:
                    fwd, bwd = f, b
                    if ps.global_rank in (ranks[0], ranks[-1]):
                        shared = sh
        _PP_GROUPS[key] = (fwd, bwd, shared)
    return _PP_GROUPS[key]
