"""Checkpoint I/O for the FSDP2 backend.

Hugging Face safetensors  <->  sharded parameters:
  * load: every engine tensor has a `LoadRecipe` (source tensors + assembly); a rank reads the sources it needs
    through memory-mapped safetensors, assembles the full local tensor and keeps its own shard
    (`Shard(0)` rows for DTensors, everything for replicated / single-rank tensors, only its experts under EP).
  * save: each parameter is gathered (`full_tensor()`), converted back to Hugging Face names and written by a
    deterministic owner rank into per-rank shard files of at most 5 GiB; expert tensors are written by the EP rank
    that owns them; the index is published last so a partial export is never mistaken for a complete one.
Native sharded state uses `torch.distributed.checkpoint`: model state includes frozen parameters, tensors that
differ per EP rank are stamped `::ep<rank>` so their keys are unique, loading ignores extra saved entries but
requires every current one (engine/backends/fsdp2/checkpoint/{dcp,weight_loader,weight_saver}.py of the reference).
"""
from __future__ import annotations

import json
import os
import shutil
from pathlib import Path
from typing import Any

import torch
import torch.distributed as dist
import torch.nn as nn

from ....logging import get_logger
from ...checkpoint.layout import DCP_COMMIT, HF_INDEX, dcp_status, fsync_dir, save_json
from ...peft.lora import is_adapter_param, lora_merge_functions, strip_peft_name
from ..base import BaseCheckpointManager

logger = get_logger(__name__)

MAX_SHARD_BYTES = int(os.environ.get("TORCHTURBO_HF_SHARD_BYTES", 5 * 1024 ** 3))


def _is_dtensor(t) -> bool:
    return hasattr(t, "_local_tensor")


def _rank() -> int:
    return dist.get_rank() if dist.is_initialized() else 0


def _world() -> int:
    return dist.get_world_size() if dist.is_initialized() else 1


class _SafetensorsReader:
    def __init__(self, root: str, tensor_files: dict[str, str]):
        self.root, self.tensor_files = Path(root), tensor_files
        self._open: dict[str, Any] = {}

    def get(self, name: str) -> torch.Tensor:
        from safetensors import safe_open

        fn = self.tensor_files.get(name)
        if fn is None:
            raise KeyError(f"tensor {name!r} is not in the checkpoint")
        if fn not in self._open:
            self._open[fn] = safe_open(str(self.root / fn), framework="pt", device="cpu")
        return self._open[fn].get_tensor(name)

    def close(self) -> None:
        self._open.clear()


class FSDP2CheckpointManager(BaseCheckpointManager):
    def __init__(self, backend) -> None:
        self.backend = backend

    # ------------------------------------------------------------------------------------------
    # Hugging Face load
    # ------------------------------------------------------------------------------------------
    def _named_state(self, model: nn.Module):
        seen: set[int] = set()
        for name, p in model.named_parameters(remove_duplicate=False):
            yield name, p, id(p) in seen
            seen.add(id(p))
        persistent = set(model.state_dict().keys())
        for name, b in model.named_buffers():
            if name in persistent:
                yield name, b, False

    @torch.no_grad()
    def load_hf(self, model: nn.Module, path: str) -> None:
        """Hugging Face safetensors -> this rank's shards.

        With more than one rank the work is split instead of repeated: every tensor that all ranks need (everything but
        expert-parallel tensors) has ONE reader rank, chosen by the shard file its first source lives in, so each file
        is opened and decoded by one rank; the reader assembles the engine tensor (fused projections, dtype cast) on
        its device and broadcasts it, and every rank cuts its own shard out of what it receives.  Broadcasts are
        asynchronous and issued in windows of at most `TORCHTURBO_LOAD_BROADCAST_BYTES` (default 5 GiB) in flight, the
        same bound the reference uses (engine/backends/fsdp2/checkpoint/weight_loader.py:68-72,232-592 there).
        Expert-parallel tensors differ per rank, so each rank reads only the experts it owns."""
        conv = model.get_weight_converter(self.backend.get_parallel_context(), path)
        files = conv.checkpoint_info.tensor_files
        reader = _SafetensorsReader(path, files)
        world, rank = _world(), _rank()
        eids = self.backend.expert_param_ids if self.backend.get_ep_info()["ep_size"] > 1 else set()
        budget = int(os.environ.get("TORCHTURBO_LOAD_BROADCAST_BYTES", 5 * 1024 ** 3))
        file_rank = {fn: i % world for i, fn in enumerate(sorted(set(files.values())))}
        missing: list[str] = []
        window: list[tuple[Any, torch.Tensor, torch.Tensor, str]] = []   # (work handle, buffer, target, name)
        in_flight = 0
        stats = {"read_here": 0, "received": 0, "direct": 0}

        def drain():
            nonlocal in_flight
            for work, buf, target, name in window:
                if work is not None:
                    work.wait()
                self._assign(target, buf, name)
            window.clear()
            in_flight = 0

        peft = bool(getattr(model, "peft_config", None))
        for name, t, dup in self._named_state(model):
            if dup:
                continue
            if peft:
                # adapters keep their initial values (the base checkpoint has none); wrapped base parameters are read
                # under the names of the unwrapped model
                if is_adapter_param(name):
                    continue
                name = strip_peft_name(name)
            recipe = conv.load_recipe(name)
            if recipe is None:
                continue  # tied alias omitted by the checkpoint
            absent = [s_ for s_ in recipe.sources if s_ not in files]
            if absent:      # decided from the index alone, so every rank skips the same tensors
                missing.append(f"{name} <- {absent[0]!r}")
                continue
            if world == 1 or id(t) in eids:
                self._assign(t, recipe.assemble([reader.get(s_) for s_ in recipe.sources]), name)
                stats["direct"] += 1
                continue
            owner = file_rank[files[recipe.sources[0]]]
            local = t._local_tensor if _is_dtensor(t) else t
            nbytes = t.numel() * local.element_size()
            if in_flight and in_flight + nbytes > budget:
                drain()
            if rank == owner:
                full = recipe.assemble([reader.get(s_) for s_ in recipe.sources])
                if tuple(full.shape) != tuple(t.shape):
                    raise ValueError(f"{name}: checkpoint shape {tuple(full.shape)} != parameter shape {tuple(t.shape)}")
                buf = full.to(device=local.device, dtype=local.dtype).contiguous()
                stats["read_here"] += 1
            else:
                buf = torch.empty(tuple(t.shape), dtype=local.dtype, device=local.device)
                stats["received"] += 1
            work = dist.broadcast(buf, src=owner, async_op=True)
            window.append((work, buf, t, name))
            in_flight += nbytes
        drain()
        reader.close()
        logger.info_rank0("HF load: rank 0 read %d tensor(s) itself, received %d, %d expert / single-rank read(s)",
                          stats["read_here"], stats["received"], stats["direct"])
        if missing:
            raise KeyError(f"checkpoint {path} lacks tensors for: {missing[:8]}{'...' if len(missing) > 8 else ''}")
        if hasattr(model, "tie_weights"):
            model.tie_weights()
        self.last_load_stats = stats

    def _assign(self, target: torch.Tensor, full: torch.Tensor, name: str) -> None:
        if _is_dtensor(target):
            from torch.distributed.tensor import Shard

            local = target._local_tensor
            piece = full
            for mesh_dim, pl in enumerate(target.placements):
                if isinstance(pl, Shard):
                    n = target.device_mesh.size(mesh_dim)
                    r = target.device_mesh.get_local_rank(mesh_dim)
                    chunks = torch.chunk(piece, n, dim=pl.dim)
                    piece = chunks[r] if r < len(chunks) else piece.narrow(pl.dim, 0, 0)
            if tuple(piece.shape) != tuple(local.shape):
                # uneven sharding: FSDP pads the last shard; copy what exists
                sl = tuple(slice(0, s) for s in piece.shape)
                local.zero_()
                local[sl].copy_(piece.to(local.dtype))
            else:
                local.copy_(piece.to(local.dtype))
        else:
            if tuple(full.shape) != tuple(target.shape):
                raise ValueError(f"{name}: checkpoint shape {tuple(full.shape)} != parameter shape {tuple(target.shape)}")
            target.copy_(full.to(target.dtype))

    # ------------------------------------------------------------------------------------------
    # Hugging Face save
    # ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def save_hf(self, model: nn.Module, path: str, *, source_path: str | None = None, dtype=torch.bfloat16) -> None:
        from safetensors.torch import save_file

        self.backend.reshard_all(model)
        ctx = self.backend.get_parallel_context()
        # with the source checkpoint at hand the export mirrors its expert format (fused 3-D tensors or per expert)
        has_src = bool(source_path) and os.path.isdir(source_path) and (
            os.path.exists(os.path.join(source_path, HF_INDEX)) or
            any(f.endswith(".safetensors") for f in os.listdir(source_path)))
        conv = model.get_weight_converter(ctx, source_path if has_src else None)
        rank, world = _rank(), _world()
        ep_size, ep_rank = ctx["ep"]["ep_size"], ctx["ep"]["ep_rank"]
        if rank == 0:
            os.makedirs(path, exist_ok=True)
        if world > 1:
            dist.barrier()
        lora = getattr(model, "merged_lora_delta", None)
        weight_map: dict[str, str] = {}

        class _Shards:
            """Accumulates tensors and writes a file whenever the next one would pass the shard size."""

            def __init__(self, stem: str):
                self.stem, self.idx, self.cur, self.bytes = stem, 0, {}, 0

            def add(self, key: str, t: torch.Tensor) -> None:
                n = t.numel() * t.element_size()
                if self.cur and self.bytes + n > MAX_SHARD_BYTES:
                    self.flush()
                self.cur[key] = t
                self.bytes += n

            def flush(self) -> None:
                if not self.cur:
                    return
                fn = f"{self.stem}-{self.idx:05d}.safetensors"
                save_file({k: v.contiguous() for k, v in self.cur.items()}, os.path.join(path, fn), metadata={"format": "pt"})
                with open(os.path.join(path, fn), "rb") as f:
                    os.fsync(f.fileno())
                for k in self.cur:
                    weight_map[k] = fn
                self.idx, self.cur, self.bytes = self.idx + 1, {}, 0

        # per-EP-rank pieces of fused expert tensors go to files of their own: rank 0 joins them and removes the files
        shards, pieces = _Shards(f"model-rank{rank:05d}"), _Shards(f"ep-pieces-rank{rank:05d}")
        owner_rr = 0
        peft = bool(getattr(model, "peft_config", None))
        merges = lora_merge_functions(model) if peft else {}
        for name, t, dup in self._named_state(model):
            if dup:
                continue
            merge = merges.get(name)
            if peft:
                # the export is a plain checkpoint of the base architecture: adapters are merged into the weights they
                # wrap and not written themselves (engine/backends/fsdp2/checkpoint/weight_saver.py:391-409 of the reference)
                if is_adapter_param(name):
                    continue
                name = strip_peft_name(name)
            is_expert = conv.is_expert_param(name)
            full = t.full_tensor() if _is_dtensor(t) else t
            master = getattr(t, "_tt_master", None)
            if master is not None:
                full = master
            if is_expert and ep_size > 1:
                # unique per EP rank: written by the member of each EP position with the lowest world rank
                writer = (rank == min(r for r in range(world) if r % ep_size == ep_rank))
            else:
                writer = (rank == owner_rr % world)
                owner_rr += 1
            if merge is not None:
                full = merge(full.detach())         # gathers the adapter factors: every rank takes part
            if not writer:
                continue
            if merge is None and lora is not None and name in lora:
                full = full.float() + lora[name].to(full.device).float()
            for hf_name, ht in conv.to_hf_tensors(name, full.detach()).items():
                ht = ht.to(dtype if ht.dtype.is_floating_point else ht.dtype).cpu()
                (pieces if "__ep" in hf_name else shards).add(hf_name, ht)
        shards.flush()
        pieces.flush()
        maps: list[dict] = [weight_map]
        if world > 1:
            maps = [None] * world
            dist.all_gather_object(maps, weight_map)
        if rank == 0:
            merged: dict[str, str] = {}
            for m in maps:
                merged.update(m)
            merged = self._merge_virtual_ep_keys(path, merged)
            if source_path and os.path.isdir(source_path):
                for fn in os.listdir(source_path):
                    src = os.path.join(source_path, fn)
                    if os.path.isfile(src) and not fn.endswith(".safetensors") and fn != HF_INDEX:
                        shutil.copy2(src, os.path.join(path, fn))
            cfg = getattr(model, "config", None)
            if cfg is not None and hasattr(cfg, "save_pretrained") and not os.path.exists(os.path.join(path, "config.json")):
                cfg.save_pretrained(path)
            fsync_dir(path)
            save_json(os.path.join(path, HF_INDEX), {"metadata": {"format": "pt"}, "weight_map": dict(sorted(merged.items()))})
        if world > 1:
            dist.barrier()

    def _merge_virtual_ep_keys(self, path: str, weight_map: dict[str, str]) -> dict[str, str]:
        """Fused-expert checkpoints write one `<name>__ep<r>` piece per EP rank; concatenate them (rank order) into
        the real tensors, written in size-bounded files one tensor at a time, and remove the piece files."""
        from safetensors import safe_open
        from safetensors.torch import save_file

        groups: dict[str, list[tuple[int, str]]] = {}
        for k in weight_map:
            if "__ep" in k:
                base, _, r = k.rpartition("__ep")
                groups.setdefault(base, []).append((int(r), k))
        if not groups:
            return weight_map
        out = {k: v for k, v in weight_map.items() if "__ep" not in k}
        cur, cur_bytes, idx = {}, 0, 0

        def flush():
            nonlocal cur, cur_bytes, idx
            if not cur:
                return
            fn = f"model-fused-experts-{idx:05d}.safetensors"
            save_file(cur, os.path.join(path, fn), metadata={"format": "pt"})
            for base in cur:
                out[base] = fn
            cur, cur_bytes, idx = {}, 0, idx + 1

        for base, parts in sorted(groups.items()):
            pcs = []
            for _, k in sorted(parts):
                with safe_open(os.path.join(path, weight_map[k]), framework="pt", device="cpu") as f:
                    pcs.append(f.get_tensor(k))
            t = torch.cat(pcs, dim=0)
            n = t.numel() * t.element_size()
            if cur and cur_bytes + n > MAX_SHARD_BYTES:
                flush()
            cur[base] = t
            cur_bytes += n
        flush()
        for fn in {weight_map[k] for parts in groups.values() for _, k in parts}:
            os.remove(os.path.join(path, fn))
        return out

    # ------------------------------------------------------------------------------------------
    # native sharded state (torch.distributed.checkpoint)
    # ------------------------------------------------------------------------------------------
    def _ep_suffix(self) -> str:
        ep = self.backend.get_ep_info()
        return f"::ep{ep['ep_rank']}" if ep["ep_size"] > 1 else ""

    def _model_state(self, model: nn.Module) -> dict[str, torch.Tensor]:
        """FQN -> tensor (DTensor or plain), frozen parameters included, EP-unique tensors stamped."""
        suf = self._ep_suffix()
        eids = self.backend.expert_param_ids
        state = {}
        for name, t, dup in self._named_state(model):
            if dup:
                continue
            key = name + suf if (suf and id(t) in eids) else name
            state[key] = t.data if isinstance(t, nn.Parameter) else t
        return state

    def save_native_model(self, model: nn.Module, path: str) -> None:
        import torch.distributed.checkpoint as dcp

        # nested under "model" like the reference's DCP layout (keys `model.<fqn>[::ep<r>]`,
        # engine/backends/fsdp2/checkpoint/dcp.py:237-268 of the reference)
        self.backend.reshard_all(model)
        dcp.save({"model": self._model_state(model)}, checkpoint_id=path)

    def load_native_model(self, model: nn.Module, path: str) -> None:
        import torch.distributed.checkpoint as dcp

        if dcp_status(path) != "complete":
            raise RuntimeError(f"{path} is not a complete native checkpoint")
        self.backend.reshard_all(model)
        state = self._model_state(model)
        self._check_ep_keys(path, state)
        dcp.load({"model": state}, checkpoint_id=path)  # in-place into the model's tensors; extra saved keys are ignored
        if hasattr(model, "tie_weights"):
            model.tie_weights()

    def _check_ep_keys(self, path: str, state: dict[str, Any]) -> None:
        from torch.distributed.checkpoint import FileSystemReader

        saved = {k[len("model."):] for k in FileSystemReader(path).read_metadata().state_dict_metadata.keys() if k.startswith("model.")}
        saved_ep = sorted({k.rpartition("::ep")[2] for k in saved if "::ep" in k})
        ep_size = self.backend.get_ep_info()["ep_size"]
        if saved_ep and len(saved_ep) != ep_size:
            # expert tensors are stored once per EP rank: another EP size cannot consume them
            raise ValueError(f"native checkpoint was written with ep_size={len(saved_ep)} (expert entries ::ep{saved_ep[0]}..::ep"
                             f"{saved_ep[-1]}), this run uses ep_size={ep_size}; export to Hugging Face format to change it")
        missing = [k for k in state if k not in saved]
        if missing:
            hint = f" (checkpoint EP ranks: {saved_ep}; current suffix {self._ep_suffix() or 'none'})" if saved_ep or self._ep_suffix() else ""
            raise KeyError(f"native checkpoint lacks {len(missing)} required entries, e.g. {missing[:4]}{hint}")

    # -- optimizer -------------------------------------------------------------------------------------
    def _flatten_optimizer(self, model: nn.Module, optimizer) -> tuple[dict[str, torch.Tensor], dict[str, Any]]:
        self.backend.reshard_all(model)
        from ...optimizers import OptimizersContainer

        names = {id(p): n for n, p in model.named_parameters()}
        suf = self._ep_suffix()
        opts = list(optimizer) if isinstance(optimizer, OptimizersContainer) else [optimizer]
        onames = optimizer.names if isinstance(optimizer, OptimizersContainer) else ["opt0"]
        tensors: dict[str, torch.Tensor] = {}
        groups: dict[str, Any] = {}
        eids = self.backend.expert_param_ids
        for oname, opt in zip(onames, opts):
            groups[oname] = [{k: v for k, v in g.items() if k != "params"} | {"params": [names[id(p)] for p in g["params"]]}
                             for g in opt.param_groups]
            self._materialize_state(opt)
            for g in opt.param_groups:
                for p in g["params"]:
                    st = opt.state.get(p, {})
                    stamp = suf if (suf and id(p) in eids) else ""
                    for k, v in st.items():
                        if isinstance(v, torch.Tensor):
                            tensors[f"{oname}/{names[id(p)]}{stamp}/{k}"] = v
        return tensors, groups

    @staticmethod
    @torch.no_grad()
    def _materialize_state(opt) -> None:
        """Make sure every trainable parameter has its state tensors (a freshly built optimizer has none, and
        loading needs destinations).  Optimizers without an explicit initialiser take one step on zero gradients
        with their parameters saved and restored around it."""
        if hasattr(opt, "_init_state"):
            for g in opt.param_groups:
                for p in g["params"]:
                    if p.requires_grad:
                        opt._init_state(p)
            return
        missing = [p for g in opt.param_groups for p in g["params"] if p.requires_grad and len(opt.state.get(p, {})) == 0]
        if not missing:
            return
        saved = [(p, (p._local_tensor if _is_dtensor(p) else p).detach().clone(), p.grad) for p in missing]
        for p in missing:
            p.grad = torch.zeros_like(p)
        others = [(p, p.grad) for g in opt.param_groups for p in g["params"] if p not in set(missing)]
        for p, _ in others:
            p.grad = None
        opt.step()
        for p, data, grad in saved:
            (p._local_tensor if _is_dtensor(p) else p).copy_(data)
            p.grad = grad
            st = opt.state[p]
            for k, v in st.items():
                if isinstance(v, torch.Tensor):
                    v.zero_()
        for p, grad in others:
            p.grad = grad

    def save_native_optimizer(self, model: nn.Module, optimizer, path: str) -> None:
        import torch.distributed.checkpoint as dcp

        tensors, groups = self._flatten_optimizer(model, optimizer)
        # keys `optimizer.state.<optimizer>/<fqn>[::ep<r>]/<slot>` and `optimizer.param_groups.<optimizer>`: nested
        # under "optimizer" like the reference's layout (dcp.py:370-388 there), one entry per state tensor
        dcp.save({"optimizer": {"state": tensors, "param_groups": groups}}, checkpoint_id=path)

    def load_native_optimizer(self, model: nn.Module, optimizer, path: str) -> None:
        import torch.distributed.checkpoint as dcp

        tensors, groups = self._flatten_optimizer(model, optimizer)
        holder = {"state": tensors, "param_groups": groups}
        dcp.load({"optimizer": holder}, checkpoint_id=path)
        from ...optimizers import OptimizersContainer

        opts = list(optimizer) if isinstance(optimizer, OptimizersContainer) else [optimizer]
        onames = optimizer.names if isinstance(optimizer, OptimizersContainer) else ["opt0"]
        for oname, opt in zip(onames, opts):
            for g, saved in zip(opt.param_groups, holder["param_groups"].get(oname, [])):
                for k, v in saved.items():
                    if k != "params":
                        g[k] = v
            # bf16 parameters follow their restored fp32 master
            for g in opt.param_groups:
                for p in g["params"]:
                    m = opt.state.get(p, {}).get("master")
                    if m is not None:
                        lp = p._local_tensor if _is_dtensor(p) else p
                        lp.data.copy_(m.to(lp.dtype))

    def native_model_status(self, path: str) -> str:
        return dcp_status(path)

    def native_optimizer_status(self, path: str) -> str:
        return dcp_status(path)
