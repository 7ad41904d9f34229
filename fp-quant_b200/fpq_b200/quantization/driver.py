"""Model-level MR-GPTQ / RTN drivers with the call signature and return value of
`gptq_quantization` (src/quantization/gptq.py:225-470) and `rtn_quantization`
(src/quantization/rtn.py:17-237) of IST-DASLab/FP-Quant.

Differences in structure (same mathematics):
  * instead of swapping the attention / MLP modules for model-specific classes, every nn.Linear of a
    transformer block is wrapped by `RotatedLinear`, which rotates its input, optionally fake-quantises
    it and multiplies by the (rotated) weight -- (x H)(W H)^T = x W^T, so the block computes the same
    function for any architecture whose blocks are built from nn.Linear;
  * linears that read the same tensor (q/k/v, gate/up) share one Hessian accumulation instead of
    accumulating identical matrices once per layer;
  * all numeric steps are the CUDA kernels of this package;
  * when torch.distributed is initialised with several ranks (one per GPU, every rank holding the same
    model), the calibration sequences are split over the ranks, the Hessians are all-reduced, the
    Cholesky-inverse chains of a block's distinct Hessians run on different ranks and their factors are
    broadcast, and every linear is quantised, whole, by one rank (`plan_ranks`) that broadcasts the
    result.  Every rank returns the full result.
"""
from __future__ import annotations

import contextlib
import re
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _cabi as C
from .. import dist as fdist
from .. import ops
from ..transforms.transforms import build_transform, get_transform_matrix
from .gptq import GPTQ, get_relative_mse_error
from .quant_args import QuantizationOrder, ScalePrecision
from .quant_ops import cast_scales_to_eXmY
from .quantizer import Quantizer


class ForwardInterrupt(Exception):
    pass


class _Phases:
    """Device time per phase of the driver (CUDA events; read with `.summary()` after a synchronise)."""

    def __init__(self):
        self.marks = []

    def mark(self, name: str) -> None:
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.marks.append((name, e))

    def summary(self) -> Dict[str, float]:
        torch.cuda.synchronize()
        out: Dict[str, float] = {}
        for (n0, e0), (n1, e1) in zip(self.marks[:-1], self.marks[1:]):
            out[n1] = out.get(n1, 0.0) + e0.elapsed_time(e1) * 1e-3
        return out


last_phases: Optional[_Phases] = None     # phases of the most recent gptq_quantization call
last_relative_mse: Dict[str, float] = {}  # "model.layers.<i>.<linear>" -> relative MSE of the most recent call (rank 0 prints them)
_split_state: dict = {}                   # per process: side stream of the split second pass; whether the split is exact for this model


class _HessianSink:
    """Collects the rotated inputs of consecutive calibration sequences and hands them to `GPTQ.update` a
    few at a time: every update reads and rewrites the whole d x d Hessian (0.8 GB for d = 14336), so one
    update per 2048-token sequence spends more time on that than on the product.  The running mean is the
    same (update counts sequences by the leading dimension)."""

    def __init__(self, handle: "GPTQ", tokens_per_update: int = 16384):
        self.handle, self.limit = handle, tokens_per_update
        self.pending: List[torch.Tensor] = []
        self.tokens = 0

    def __call__(self, x: torch.Tensor) -> None:
        x = x if x.dim() >= 3 else x.unsqueeze(0)
        if self.pending and self.pending[0].shape[1:] != x.shape[1:]:
            self.flush()
        self.pending.append(x)
        self.tokens += x.numel() // x.shape[-1]
        if self.tokens >= self.limit:
            self.flush()

    def flush(self) -> None:
        if self.pending:
            self.handle.update(self.pending[0] if len(self.pending) == 1 else torch.cat(self.pending, dim=0))
        self.pending, self.tokens = [], 0


class InputCollector(nn.Module):
    """Records the positional and keyword inputs of the wrapped block and stops the forward pass
    (src/utils/model_utils.py:19-38)."""

    def __init__(self, module: nn.Module, cpu_offload: bool = False):
        super().__init__()
        self.module, self.cpu_offload = module, cpu_offload
        self.input_args, self.input_kwargs = [], []

    def forward(self, *args, **kwargs):
        if self.cpu_offload:
            args, kwargs = _to(args, "cpu"), _to(kwargs, "cpu")
        self.input_args.append(args)
        self.input_kwargs.append(kwargs)
        raise ForwardInterrupt


def _to(obj, device):
    if isinstance(obj, torch.Tensor):
        return obj.to(device)
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to(o, device) for o in obj)
    if isinstance(obj, dict):
        return {k: _to(v, device) for k, v in obj.items()}
    return obj


def _first(x):
    return x[0] if isinstance(x, (list, tuple)) else x


class RotatedLinear(nn.Module):
    """y = fake_quant(rotate(x)) @ rotate(W)^T + b.  While `_train_mode` the weight is rotated on the
    fly (it is still the original); afterwards it holds the rotated, quantised weight.

    Linears that are fed the same tensor (q/k/v, gate/up) share `group_state`: the first of them to see a
    tensor rotates and fake-quantises it, the others reuse the result (same activation quantiser, so the
    numbers are the ones each would have computed)."""

    def __init__(self, linear: nn.Linear, transform, act_quantizer: Optional[Quantizer], group_state: Optional[dict] = None):
        super().__init__()
        self.weight, self.bias = linear.weight, linear.bias
        self.in_features, self.out_features = linear.in_features, linear.out_features
        self.transform, self.act_quantizer = transform, act_quantizer
        self._train_mode = True
        self.input_sink = None          # called with the rotated, unquantised input (Hessian accumulation)
        self.group_state = group_state if group_state is not None else {}
        self._rotated = None            # (weight version, rotated weight) while the weight is still the original
        self.deferred_inputs = None     # a list: forward() stores its prepared input there and returns zeros

    def _prepared_input(self, x: torch.Tensor) -> torch.Tensor:
        st = self.group_state
        if st.get("x") is x and st.get("version") == x._version:
            return st["xq"]
        xr = self.transform(x)
        if st.get("sink") is not None:
            st["sink"](xr)
        xq = xr
        if self.act_quantizer is not None:
            xq = self.act_quantizer.fused_fake_quantize(xr, hadamard_group=0, ste=False)
        st["x"], st["version"], st["xq"] = x, x._version, xq
        return xq

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.input_sink is not None:          # legacy hook of a stand-alone module
            self.group_state["sink"] = self.input_sink
        xq = self._prepared_input(x)
        if self.deferred_inputs is not None:      # first half of a split pass: the product is added later
            self.deferred_inputs.append(xq)
            return xq.new_zeros(*xq.shape[:-1], self.out_features)
        if self._train_mode:
            # the same weight is rotated for every calibration sequence: keep the result until the weight changes
            if self._rotated is None or self._rotated[0] != self.weight._version:
                self._rotated = (self.weight._version, self.transform(self.weight, inv_t=True))
            w = self._rotated[1]
        else:
            self._rotated = None
            w = self.weight
        return F.linear(xq, w, self.bias)


# linears that are fed the same tensor share a Hessian
_INPUT_GROUPS = (("qkv", r"(q|k|v)_proj$"), ("o", r"o_proj$"), ("gate_up", r"(gate|up)_proj$"), ("down", r"down_proj$"))


def _input_group(name: str) -> str:
    for key, pat in _INPUT_GROUPS:
        if re.search(pat, name):
            return key
    return name


def _quantizer_kwargs(args, prefix: str) -> Optional[dict]:
    bits = getattr(args, f"{prefix}_bits")
    if bits >= 16:
        return None
    return dict(bits=bits, symmetric=True, format=args.format, granularity=getattr(args, f"{prefix}_granularity"),
                observer=getattr(args, f"{prefix}_observer"), group_size=getattr(args, f"{prefix}_group_size"),
                scale_precision=args.scale_precision)


def _wrap_block(block: nn.Module, args, device) -> Dict[str, RotatedLinear]:
    akw = _quantizer_kwargs(args, "a")
    wrapped = {}
    states: Dict[str, dict] = {}
    quantizers: Dict[str, Optional[Quantizer]] = {}
    for name, module in list(block.named_modules()):
        if isinstance(module, nn.Linear):
            parent = block
            *path, leaf = name.split(".")
            for p in path:
                parent = getattr(parent, p)
            t = build_transform(args.transform_class, size=module.in_features, device=device,
                                group_size=args.hadamard_group_size)
            grp = ".".join(path + [_input_group(leaf)])          # same parent module, same input
            if grp not in states:
                states[grp] = {}
                quantizers[grp] = Quantizer(**akw) if akw else None
            r = RotatedLinear(module, t, quantizers[grp], states[grp])
            setattr(parent, leaf, r)
            wrapped[name] = r
    return wrapped


def _release_group_states(layers: Dict[str, "RotatedLinear"]) -> None:
    for layer in layers.values():
        layer.group_state.pop("x", None)
        layer.group_state.pop("xq", None)


class _HostCopies:
    """Device -> host copies of the export tensors without stalling the stream: every tensor goes to a
    page-locked destination with an asynchronous copy, and `finish()` synchronises once.  Measured on the
    model-level benchmark (per transformer block): plain `.cpu()` per layer 48 ms; this 3 ms of copies plus
    the page-locking; a worker thread doing the same blocked the kernel launches of the next block's
    Cholesky chain (+100 ms); keeping everything on the device and copying to pageable memory at the end
    moved 220 MB at 2 GB/s (+55 ms)."""

    def __init__(self, device):
        self.device = device

    def put(self, entry: dict, key: str, tensor: torch.Tensor) -> None:
        """entry[key] becomes the host copy of `tensor` (which must not be modified afterwards)."""
        if not tensor.is_cuda:
            entry[key] = tensor
            return
        out = torch.empty(tensor.shape, dtype=tensor.dtype, pin_memory=True)
        out.copy_(tensor, non_blocking=True)
        entry[key] = out

    def finish(self) -> None:
        if torch.cuda.is_available():
            torch.cuda.synchronize()


_matrix_cache: Dict[tuple, torch.Tensor] = {}


def _export_entry(copies: _HostCopies, args, orig_dtype, device, weight_gs, act_gs, **tensors) -> dict:
    key = (str(args.transform_class), args.hadamard_group_size, str(orig_dtype))
    if key not in _matrix_cache:
        _matrix_cache[key] = get_transform_matrix(args.transform_class, args.hadamard_group_size, device, orig_dtype).cpu()
    m = _matrix_cache[key].clone()
    entry: dict = {}
    for k, v in tensors.items():
        copies.put(entry, k, v.contiguous())
    entry.update({"forward_hadamard_matrix": m, "backward_hadamard_matrix": m.clone(),
                  "weight_global_scale": weight_gs.clone(), "act_global_scale": act_gs.clone()})
    return entry


def _collect_block_inputs(model, calibration_data, args, device):
    blocks = model.model.layers
    blocks[0] = InputCollector(blocks[0], cpu_offload=args.cpu_offload_activations)
    for sample in calibration_data:
        try:
            with torch.no_grad():
                model(sample.to(device=device))
        except ForwardInterrupt:
            pass
    collector = blocks[0]
    blocks[0] = collector.module
    return collector.input_args, collector.input_kwargs


def _run_block(block, input_args, input_kwargs, device, args, keep_outputs: bool, offload_device):
    """Runs the block over the recorded calibration inputs (gptq.py:389-393, 446-457).  With
    `args.calibration_batch` > 1 several sequences go through the block in one call (their hidden states
    concatenated along the batch dimension, the other arguments taken from the first of them, which must
    therefore be the same for all sequences: no padding masks): fewer, larger launches.  The Hessian is
    unchanged by this (a sum over sequences); the activation quantiser's running-minimum tensor scale
    then advances per batch instead of per sequence."""
    batch = max(1, int(getattr(args, "calibration_batch", 1)))
    n = len(input_args)
    for i0 in range(0, n, batch):
        idx = list(range(i0, min(i0 + batch, n)))
        a0, kw0 = input_args[i0], input_kwargs[i0]
        if len(idx) == 1:
            call_args, call_kw = _to(a0, device), _to(kw0, device)
        elif len(a0) > 0:
            hs = torch.cat([_to(input_args[i][0], device) for i in idx], dim=0)
            call_args, call_kw = (hs,) + tuple(_to(a0[1:], device)), _to(kw0, device)
        elif "hidden_states" in kw0:
            call_kw = dict(_to(kw0, device))
            call_kw["hidden_states"] = torch.cat([_to(input_kwargs[i]["hidden_states"], device) for i in idx], dim=0)
            call_args = ()
        else:
            raise ValueError("Unsupported block input format.")
        with torch.no_grad(), torch.amp.autocast(device_type="cuda", enabled=getattr(args, "amp", False)):
            out = block(*call_args, **call_kw)
        if keep_outputs:
            out = _first(out).to(offload_device)
            rows = [x.shape[0] for x in ([input_args[i][0] for i in idx] if len(a0) > 0
                                        else [input_kwargs[i]["hidden_states"] for i in idx])]
            for i, piece in zip(idx, torch.split(out, rows, dim=0)):
                if len(a0) > 0:
                    input_args[i][0].data = piece
                else:
                    input_kwargs[i]["hidden_states"] = piece


def _split_pass_first_half(block, input_args, input_kwargs, device, args, last_linear: "RotatedLinear"):
    """The second pass over the calibration sequences (gptq.py:446-457) up to the input of `last_linear`, the
    block's final linear (an MLP's down-projection): every sequence goes through the block with that layer
    returning zeros, so what comes out is the residual stream the layer's output is added to.  Returns the
    per-sequence pairs (block output without the layer, the layer's prepared input).  Used on several GPUs,
    where the final linear's weight arrives last: everything that does not need it is done while its owner
    still works on it."""
    parts = []
    last_linear.deferred_inputs = []
    try:
        for a, kw in zip(input_args, input_kwargs):
            with torch.no_grad(), torch.amp.autocast(device_type="cuda", enabled=getattr(args, "amp", False)):
                out = _first(block(*_to(a, device), **_to(kw, device)))
            assert len(last_linear.deferred_inputs) == 1, "the deferred linear must run exactly once per block call"
            parts.append((out, last_linear.deferred_inputs.pop()))
    finally:
        last_linear.deferred_inputs = None
    return parts


def _split_pass_second_half(parts, input_args, input_kwargs, last_linear: "RotatedLinear", offload_device) -> None:
    """Adds the final linear's product to the stored residual streams and writes the block outputs where
    `_run_block(keep_outputs=True)` writes them.  bf16(residual + bf16(linear)) is the operation the block
    itself performs, so the result is bit-identical to the unsplit pass for blocks that end in
    `residual + down_proj(...)` (`_split_pass_is_exact` checks that on the first sequence)."""
    for (out, xq), a, kw in zip(parts, input_args, input_kwargs):
        y = out + F.linear(xq, last_linear.weight, last_linear.bias)
        y = y.to(offload_device)
        if len(a) > 0:
            a[0].data = y
        elif "hidden_states" in kw:
            kw["hidden_states"] = y
        else:
            raise ValueError("Unsupported block input format.")


def _split_pass_is_exact(block, parts, input_args, input_kwargs, device, args, last_linear) -> bool:
    """Whether the split pass reproduces the block on the first sequence bit for bit (weights final)."""
    with torch.no_grad(), torch.amp.autocast(device_type="cuda", enabled=getattr(args, "amp", False)):
        want = _first(block(*_to(input_args[0], device), **_to(input_kwargs[0], device)))
    out, xq = parts[0]
    return bool(torch.equal(want, out + F.linear(xq, last_linear.weight, last_linear.bias)))


def plan_ranks(group_members: Dict[str, List[str]], group_cols: Dict[str, int], world_size: int):
    """Which rank factors which Hessian and quantises which linear of a block.

    group_members: input group -> its linears (the first is the group's leader); group_cols: input width of
    the group (the Cholesky chain costs ~ width^3).  Returns (groups ordered by cost, group -> rank that runs
    its chain, linear -> rank that runs its column loop).  Chains go round-robin, largest first; a group's
    leader stays on the chain's rank (no transfer of U needed), the other members move to ranks that have
    no chain, while there are any."""
    group_order = sorted(group_members, key=lambda g: -group_cols[g])
    group_owner = {g: i % world_size for i, g in enumerate(group_order)}
    idle = [r for r in range(world_size) if r not in set(group_owner.values())]
    layer_owner: Dict[str, int] = {}
    for g in group_order:
        for k, n in enumerate(group_members[g]):
            layer_owner[n] = group_owner[g] if (k == 0 or not idle) else idle.pop(0)
    return group_order, group_owner, layer_owner


@torch.no_grad()
def gptq_quantization(model, calibration_data: List[torch.Tensor], args, device) -> Tuple[dict, dict]:
    """MR-GPTQ over the transformer blocks of `model` (gptq.py:225-470).  Returns
    (quantized_state_dict, non_quantized_state_dict) with the reference's per-layer keys."""
    if fdist.world()[0] == 0:
        print("GPTQ quantization...")
    orig_dtype = model.config.torch_dtype if args.dtype == "auto" else args.dtype
    offload = "cpu" if args.cpu_offload_activations else device
    quantized, non_quantized = {}, {}
    wkw = _quantizer_kwargs(args, "w")
    global last_phases
    ph = last_phases = _Phases()
    last_relative_mse.clear()
    pending_mse: Dict[str, torch.Tensor] = {}
    copies = _HostCopies(device)
    ph.mark("start")
    rank, world_size = fdist.world()
    n_total = len(calibration_data)
    # Rank 0 gets the widest Hessian's chain and column loop (`plan_ranks`), which the other ranks wait for once
    # they have run the second pass up to that layer; its own share of that pass runs after them.  It is
    # therefore given fewer calibration sequences, so that its forward passes fit into the time the others
    # need for theirs.  The shares were balanced on a Llama-3.1-8B block with 128 x 2048 tokens (0.82 / 0.6 /
    # 0.45 of an even share at 2 / 4 / 8 ranks; at 8 ranks 0.25, 0.45 and 0.62 gave 0.111, 0.107 and 0.110 s per
    # block); `args.owner_share` overrides them, 1.0 is an even split.
    share = getattr(args, "owner_share", None)
    if share is None:
        share = {2: 0.82, 4: 0.6, 8: 0.45}.get(world_size, 1.0 if world_size < 2 else 0.6)
    if world_size > 1 and getattr(args, "split_second_pass", True):
        rest = (world_size - share) / (world_size - 1)
        lo, hi = fdist.weighted_bounds(n_total, [share] + [rest] * (world_size - 1))[rank]
    else:
        lo, hi = fdist.shard_bounds(n_total, world_size, rank)
    n_local = hi - lo
    input_args, input_kwargs = _collect_block_inputs(model, calibration_data[lo:hi], args, device)
    ph.mark("collect_inputs")

    for block_idx, block in enumerate(model.model.layers):
        if rank == 0:
            print(f"Processing block {block_idx}...")
        block.to(device=device, dtype=orig_dtype).requires_grad_(False)
        layers = _wrap_block(block, args, device)

        # one GPTQ handle per linear; one Hessian per distinct input
        handles: Dict[str, GPTQ] = {}
        leaders: Dict[str, str] = {}
        for name, layer in layers.items():
            handles[name] = GPTQ(layer, Quantizer(**wkw) if wkw else None, quantization_order=args.quantization_order,
                                 rel_damp=args.rel_damp, export_quantized_model=args.export_quantized_model)
            handles[name].use_cuda_graphs = bool(getattr(args, "cuda_graphs", True))
            if args.scale_precision == ScalePrecision.E4M3:        # fix the weight global scale now (gptq.py:343-358)
                handles[name].quantizer.get_quantization_params(layer.transform(layer.weight, inv_t=True).float())
                handles[name].quantizer._track_global_scale = False
            grp = _input_group(name.split(".")[-1])
            if grp not in leaders:
                leaders[grp] = name
                layer.group_state["sink"] = _HessianSink(handles[name])
        if getattr(args, "fuse_global_scale", False) and args.scale_precision == ScalePrecision.E4M3:
            _fuse_weight_global_scales({n: h.quantizer for n, h in handles.items()}, device)

        ph.mark("setup")
        _run_block(block, input_args, input_kwargs, device, args, keep_outputs=False, offload_device=offload)   # Hessians
        for layer in layers.values():
            sink = layer.group_state.get("sink")
            if isinstance(sink, _HessianSink):
                sink.flush()
        ph.mark("hessian_pass")

        for name, layer in layers.items():
            layer.input_sink = None
            layer.group_state["sink"] = None
            cached = layer._rotated
            layer.weight.data = (cached[1] if cached is not None and cached[0] == layer.weight._version
                                 else layer.transform(layer.weight, inv_t=True))      # rotate once (gptq.py:395-401)
            layer._rotated = None
            layer._train_mode = False
            if layer.act_quantizer is not None:
                layer.act_quantizer._track_global_scale = False

        # ---- who does what.  One Cholesky-inverse chain per distinct Hessian when no linear of the group has an
        # all-zero weight column (the dead-column fix of gptq.py:203-208 is then the identity and the damped H,
        # hence U, is the same for all of them).  The chains go to different ranks, largest first; every linear
        # is quantised, whole, by one rank (the column loop is bound by the latency of its dependent steps, not
        # by the number of rows): the leader of a group stays with the rank that factors its Hessian, the other
        # members move to idle ranks when there are any.  Results are broadcast.
        group_members: Dict[str, List[str]] = {}
        for name in handles:
            group_members.setdefault(_input_group(name.split(".")[-1]), []).append(name)
        # (In activation order every layer permutes, damps and factors its own copy of the Hessian inside
        # `GPTQ.step`: no sharing.)
        act_order = QuantizationOrder(args.quantization_order) == QuantizationOrder.ACTIVATION
        share_ok = {grp: not act_order and
                    not any(bool((handles[n].layer.weight == 0).all(dim=0).any().item()) for n in names)
                    for grp, names in group_members.items()}
        group_order, group_owner, layer_owner = plan_ranks(
            group_members, {g: handles[leaders[g]].d_col for g in group_members}, world_size)

        # ---- the block's final linear on several GPUs.  `down_proj` has the widest Hessian (its chain and its
        # column loop take longer than everything else in the block together) and nothing else waits for it
        # but the end of the second pass.  Its owner therefore works on it on a side stream while all ranks
        # (the owner included, on its main stream, for the cheap parts) exchange the other six linears and run
        # the second pass up to the input of down_proj; the product with the finished weight is added last.
        deferred = None
        if world_size > 1 and max(1, int(getattr(args, "calibration_batch", 1))) == 1 and getattr(args, "split_second_pass", True) \
                and _split_state.get("exact", True):
            lasts = [n for n in handles if re.search(r"down_proj$", n)]
            if len(lasts) == 1 and len(group_members[_input_group(lasts[0].split(".")[-1])]) == 1:
                deferred = lasts[0]
        main_stream = torch.cuda.current_stream(device)
        side_stream = None
        if deferred is not None and layer_owner[deferred] == rank:
            if "stream" not in _split_state:
                _split_state["stream"] = torch.cuda.Stream(device=device)
            side_stream = _split_state["stream"]

        @contextlib.contextmanager
        def on_stream_of(name):
            """The side stream for the deferred linear on its owner (ordered after everything queued on the main
            stream so far), the current stream otherwise."""
            if name == deferred and side_stream is not None:
                side_stream.wait_stream(main_stream)
                with torch.cuda.stream(side_stream):
                    yield
            else:
                yield

        checks: List[torch.Tensor] = []
        shared_U: Dict[str, torch.Tensor] = {}
        chains_queued = set()

        def queue_chain(g):
            """Queues the Cholesky-inverse chain of group g's Hessian on its owner (once)."""
            if g in chains_queued:
                return
            chains_queued.add(g)
            lead = handles[leaders[g]]
            if any(layer_owner[n] == rank for n in group_members[g]):
                lead.H_undamped = lead.H.clone()
            if not share_ok[g]:
                return
            owner = group_owner[g]
            elsewhere = any(layer_owner[n] != owner for n in group_members[g])
            if rank == owner:
                timed = not (leaders[g] == deferred and side_stream is not None)    # the phase marks follow the main stream
                with on_stream_of(leaders[g]):
                    lead.defer_host_syncs = world_size > 1
                    lead.quantization_pre_step()
                    lead.prepare_hessian()
                    if timed:
                        ph.mark("factor_prepare")
                    shared_U[g] = lead._get_hessian_inverse(prepared=True)
                    if timed:
                        ph.mark("factor_chain")
            elif elsewhere:
                shared_U[g] = torch.empty((lead.d_col, lead.d_col), device=device, dtype=torch.float32)

        # ---- multi-GPU: one Hessian per distinct input, summed over the ranks' sequences, widest first.  A
        # Hessian whose linears all stay on the rank that factors it is only needed there: it is reduced to
        # that rank (half the traffic of an all-reduce), and the deferred linear's chain starts on its owner's
        # side stream as soon as its sum has arrived, under the remaining collectives.
        if world_size > 1:
            for grp in group_order:
                h = handles[leaders[grp]]
                if h.H is None:
                    h.H = torch.zeros((h.d_col, h.d_col), device=device, dtype=torch.float32)
                h.H.mul_(float(n_local) / float(n_total))     # local running mean -> this rank's share of the global mean
                if all(layer_owner[n] == group_owner[grp] for n in group_members[grp]):
                    fdist.reduce_sum_(h.H, group_owner[grp])
                else:
                    fdist.allreduce_sum_(h.H)
                h.num_samples = n_total
                if deferred is not None and leaders[grp] == deferred:
                    queue_chain(grp)
            for layer in layers.values():
                if layer.act_quantizer is not None and layer.act_quantizer.global_scale.numel() == 1:
                    gs = layer.act_quantizer.global_scale.to(device)
                    layer.act_quantizer.global_scale = fdist.allreduce_min_(gs)

        ph.mark("allreduce")
        for g in group_order:
            queue_chain(g)
        for g in group_order:                       # after all chains were queued: they overlap across ranks
            if share_ok[g] and world_size > 1 and any(layer_owner[n] != group_owner[g] for n in group_members[g]):
                torch.distributed.broadcast(shared_U[g], src=group_owner[g])

        ph.mark("factor")
        results = {}
        originals = {}
        for name, handle in handles.items():
            if layer_owner[name] != rank:
                continue
            grp = _input_group(name.split(".")[-1])
            leader = handles[leaders[grp]]
            with on_stream_of(name):
                if world_size > 1:
                    handle.defer_host_syncs = True
                    handle.quantizer.deferred_checks = checks
                if grp in shared_U and share_ok[grp]:
                    if not (handle is leader and rank == group_owner[grp]):     # the factoring rank's leader is prepared
                        handle.H, handle.num_samples = leader.H_undamped.clone(), leader.num_samples
                        handle.quantization_pre_step()
                        handle.prepare_hessian()       # same damping as the leader's: leaves the damped H for the MSE
                    wq, qweight, scales = handle.step(shared_U[grp], want_grid_values=False)   # the packed codes are exported
                else:
                    if handle is not leader:
                        handle.H, handle.num_samples = leader.H_undamped.clone(), leader.num_samples
                    wq, qweight, scales = handle.quantize(want_grid_values=False)
                if name == deferred:
                    rel = None                        # measured after the second pass, off the other ranks' path
                    originals[name] = handle.layer.weight.data
                else:
                    rel = get_relative_mse_error(wq.float(), handle.layer.weight.float(), handle.H).reshape(1)
                results[name] = (wq, handle.packed_codes, scales.float().contiguous(), rel)
        shared_U.clear()

        def exchange(name):
            """Broadcast of one linear's result from its owner (same order on every rank), weight swap, export."""
            handle = handles[name]
            rows, cols = handle.d_row, handle.d_col
            if name in results:
                wq, codes, scales, rel = results[name]
            else:
                wq = torch.empty((rows, cols), device=device, dtype=handle.W_dtype)
                codes = torch.empty((rows, cols // 2), device=device, dtype=torch.uint8)
                scales = torch.empty((rows, cols // handle.quantizer.group_size), device=device, dtype=torch.float32)
                rel = torch.empty(1, device=device, dtype=torch.float32)
            if world_size > 1:
                for t in ((wq, codes, scales) if name == deferred else (wq, codes, scales, rel)):
                    torch.distributed.broadcast(t, src=layer_owner[name])
            if rel is not None:
                pending_mse[f"model.layers.{block_idx}.{name}"] = rel
            handle.layer.weight.data = wq
            if args.export_quantized_model:
                wgs = handle.quantizer.global_scale.to(device)
                ags = handle.layer.act_quantizer.global_scale if handle.layer.act_quantizer is not None else torch.ones(1)
                key = f"model.layers.{block_idx}.{name}"
                if args.export_quantized_model == "realquant":
                    quantized[key] = _export_entry(copies, args, orig_dtype, device, wgs, ags, qweight=codes,
                                                   scales=cast_scales_to_eXmY(scales * wgs, args.scale_precision))
                else:
                    quantized[key] = _export_entry(copies, args, orig_dtype, device, wgs, ags, dqweight=wq)

        for name in handles:                        # same order on every rank: one broadcast group per linear
            if name != deferred:
                exchange(name)
        ph.mark("column_loops")
        _release_group_states(layers)
        if deferred is None:
            _run_block(block, input_args, input_kwargs, device, args, keep_outputs=True, offload_device=offload)
        else:
            last = handles[deferred].layer
            if side_stream is not None:
                # The owner's own sequences wait for its side stream (its forward kernels would only slow the
                # chain and the loop down), and the finished weight goes out before they run: the other ranks
                # wait for the weight, not for the owner's share of the pass.  (Same order of collectives on
                # every rank; only their place among the local launches differs.)
                main_stream.wait_stream(side_stream)
                exchange(deferred)
                parts = _split_pass_first_half(block, input_args, input_kwargs, device, args, last)
            else:
                parts = _split_pass_first_half(block, input_args, input_kwargs, device, args, last)
                exchange(deferred)
            ph.mark("update_pass_first_half")
            if "exact" not in _split_state:      # once per process: does this architecture end in residual + down_proj?
                mine = (not parts) or _split_pass_is_exact(block, parts, input_args, input_kwargs, device, args, last)
                verdict = torch.tensor([1 if mine else 0], device=device, dtype=torch.int32)
                torch.distributed.all_reduce(verdict, op=torch.distributed.ReduceOp.MIN)    # one answer for all ranks
                _split_state["exact"] = bool(verdict.item())
            if _split_state["exact"]:
                _split_pass_second_half(parts, input_args, input_kwargs, last, offload)
            else:
                _run_block(block, input_args, input_kwargs, device, args, keep_outputs=True, offload_device=offload)
            del parts
            if deferred in results:              # the owner measures its layer now that nobody waits for it
                handle = handles[deferred]
                pending_mse[f"model.layers.{block_idx}.{deferred}"] = get_relative_mse_error(
                    results[deferred][0].float(), originals[deferred].float(), handle.H).reshape(1)
            elif rank == 0:
                pending_mse[f"model.layers.{block_idx}.{deferred}"] = torch.full((1,), float("nan"), device=device)
        results.clear()
        originals.clear()
        _release_group_states(layers)
        ph.mark("update_pass")
        # one host read per block: finiteness checks of the quantisers and the log line of every layer (gptq.py:414-415)
        if checks and bool(torch.stack([c.reshape(()) for c in checks]).any().item()):
            raise ValueError("Scales or global scale are not finite.")
        names = [k for k in pending_mse if k not in last_relative_mse]
        if names:
            values = torch.cat([pending_mse[k] for k in names]).tolist()
            for k, v in zip(names, values):
                last_relative_mse[k] = v
                if rank == 0:
                    print(f"[{k.split('.', 3)[3]:16}]: Relative MSE error: {v:.2e}")
        if getattr(args, "cpu_offload_modules", False):
            block.cpu()
        del handles
    copies.finish()                       # the background copies of the export tensors have landed
    return quantized, non_quantized


def _fuse_weight_global_scales(quantizers: Dict[str, Quantizer], device) -> None:
    """q/k/v and gate/up share the smallest of their weight tensor scales (gptq.py:367-383, rtn.py:134-150)."""
    for pat in (r"(q|k|v)_proj$", r"(gate|up)_proj$"):
        names = [n for n in quantizers if re.search(pat, n)]
        if names:
            fused = torch.stack([quantizers[n].global_scale.to(device) for n in names]).min(dim=0).values
            for n in names:
                quantizers[n].global_scale = fused.clone()


@torch.no_grad()
def rtn_quantization(model, calibration_data: List[torch.Tensor], args, device) -> Tuple[dict, dict]:
    """Round-to-nearest over all blocks (rtn.py:17-237).  Per block: fix (and optionally fuse) the weight
    tensor scales, quantise every rotated weight with its quantiser (min-max or MSE observer), and -- when
    the scales are E4M3, i.e. the format has an activation tensor scale that must be settled on data
    (rtn.py:26) -- run the calibration sequences through the block once so that the activation quantisers
    see every input (rtn.py:152-156), freeze them, export, and run the sequences again to produce the next
    block's inputs (rtn.py:216-228).

    The reference's first pass computes with the fake-quantised rotated weight rebuilt on the fly and
    `fix_parametrization` stores that same weight afterwards (qlinear.py:36-47, :52-76); here the weight is
    quantised once, before the first pass, which feeds both passes the identical matrix."""
    print("RTN quantization...")
    orig_dtype = model.config.torch_dtype if args.dtype == "auto" else args.dtype
    offload = "cpu" if args.cpu_offload_activations else device
    need_calibration = args.scale_precision == ScalePrecision.E4M3
    quantized, non_quantized = {}, {}
    copies = _HostCopies(device)
    wkw = _quantizer_kwargs(args, "w")
    input_args = input_kwargs = None
    if need_calibration:
        input_args, input_kwargs = _collect_block_inputs(model, calibration_data, args, device)
    for block_idx, block in enumerate(model.model.layers):
        print(f"Processing block {block_idx}...")
        block.to(device=device, dtype=orig_dtype).requires_grad_(False)
        layers = _wrap_block(block, args, device)
        rotated = {name: layer.transform(layer.weight, inv_t=True) for name, layer in layers.items()}
        wq: Dict[str, Quantizer] = {}
        if wkw:
            wq = {name: Quantizer(**wkw) for name in layers}
            if need_calibration:                                   # rtn.py:116-131: set and freeze the tensor scales
                for name, q in wq.items():
                    q.get_quantization_params(rotated[name].float())
                    q._track_global_scale = False
                if getattr(args, "fuse_global_scale", False):
                    _fuse_weight_global_scales(wq, device)
        exports = {}
        for name, layer in layers.items():
            w = rotated[name]
            if name in wq:
                q = wq[name]
                group = q.group_size
                scales, _ = q.get_quantization_params(w.float())             # honours the observer (rtn.py:175)
                scales = scales.float().contiguous()
                codes = ops.apply_scales(w.float(), scales, group, C.OUT_CODES)
                layer.weight.data = ops.apply_scales(w.float(), scales, group, C.OUT_DEQUANT).to(w.dtype)
                exports[name] = (codes, scales, q.global_scale.to(device))
            else:
                layer.weight.data = w
            layer._rotated = None
            layer._train_mode = False
        del rotated

        if need_calibration:
            _run_block(block, input_args, input_kwargs, device, args, keep_outputs=False, offload_device=offload)
            _release_group_states(layers)
        for layer in layers.values():
            if layer.act_quantizer is not None:
                layer.act_quantizer._track_global_scale = False

        if args.export_quantized_model:
            for name, layer in layers.items():
                if name not in exports:
                    continue
                codes, scales, wgs = exports[name]
                ags = layer.act_quantizer.global_scale if layer.act_quantizer is not None else torch.ones(1)
                key = f"model.layers.{block_idx}.{name}"
                if args.export_quantized_model == "realquant":
                    quantized[key] = _export_entry(copies, args, orig_dtype, device, wgs, ags, qweight=codes,
                                                   scales=cast_scales_to_eXmY(scales * wgs, args.scale_precision))
                else:
                    quantized[key] = _export_entry(copies, args, orig_dtype, device, wgs, ags, dqweight=layer.weight.data)
        exports.clear()

        if need_calibration:
            _run_block(block, input_args, input_kwargs, device, args, keep_outputs=True, offload_device=offload)
            _release_group_states(layers)
        if getattr(args, "cpu_offload_modules", False):
            block.cpu()
    copies.finish()
    return quantized, non_quantized
