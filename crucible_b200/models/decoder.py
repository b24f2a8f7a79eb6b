"""The generic decoder: embedding, a list of layers built from registered parts,
a run order over them, a final norm and an LM head.

Nothing here is specific to one architecture: the `ModelConfig` says which
part kinds each layer has and in which order the layers run.  From the mixers'
cache needs it derives the cache groups (layers whose needs are identical share
pages and a block table; layers with a window get pages of their own) and each
run-order entry's binding.

Forward order follows `engine/src/gpu_model.rs:3254-3580` (prefill) and
`:1393-1605` (decode): embed -> layers -> gather wanted rows -> final norm ->
LM head.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from .. import ops
from ..config.model_config import ConfigError, ModelConfig
from ..parts import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, CacheNeed,
                     LayerBinding, TensorDecl)


@dataclass(frozen=True)
class CacheGroupSpec:
    """Layers whose keys and values share pages: one pool, one block table."""
    need: CacheNeed
    layers: Tuple[int, ...]          # stored-layer indices, in slot order


@dataclass(frozen=True)
class TensorRequest:
    key: str                         # "<part path>.<local name>", unique in the model
    checkpoint_name: str
    decl: TensorDecl


class DecoderModel:
    def __init__(self, config: ModelConfig):
        self.config = config
        self.embedding = EMBEDDINGS.build(config.embedding.kind, config.embedding,
                                          config.vocab_size, config.hidden_size)
        self.head = HEADS.build(config.head.kind, config.head, config.vocab_size,
                                config.hidden_size, config.tie_word_embeddings)
        self.final_norm = NORMS.build(config.final_norm.kind, config.final_norm)
        self.layers = []
        for spec in config.layers:
            mixer = MIXERS.build(spec.mixer.kind, spec.mixer)
            ffn = FEED_FORWARDS.build(spec.feed_forward.kind, spec.feed_forward)
            norms = {name: NORMS.build(n.kind, n) for name, n in spec.norms}
            self.layers.append(ARRANGEMENTS.build(spec.arrangement, spec, norms, mixer, ffn))
        self.cache_groups, self.bindings, self.state_bytes = self._plan_storage()
        self.dtype: Optional[torch.dtype] = None
        self.device: Optional[torch.device] = None

    # -- storage planning ---------------------------------------------------

    def _plan_storage(self):
        """Cache groups, one binding per run-order entry, state bytes per request."""
        owners: Dict[int, Tuple[int, int]] = {}       # stored layer -> (group, slot)
        groups: List[Tuple[CacheNeed, List[int]]] = []
        for li, layer in enumerate(self.layers):
            need = layer.mixer.cache_need()
            if need is None:
                continue
            for gi, (gneed, members) in enumerate(groups):
                if gneed == need:
                    owners[li] = (gi, len(members))
                    members.append(li)
                    break
            else:
                owners[li] = (len(groups), 0)
                groups.append((need, [li]))
        bindings: List[LayerBinding] = []
        state_offsets: Dict[int, int] = {}
        total_state = 0
        written = set()
        for i, entry in enumerate(self.config.run_order):
            layer = self.layers[entry.layer]
            nbytes = int(layer.mixer.state_bytes())
            if nbytes and entry.layer not in state_offsets:
                state_offsets[entry.layer] = total_state
                total_state += (nbytes + 15) // 16 * 16
            group = slot = None
            write = True
            if entry.cache_of is not None:
                src = entry.cache_of
                if src not in owners:
                    raise ConfigError(f"run_order[{i}] reads the cache of layer {src}, "
                                      f"whose mixer keeps none")
                if layer.mixer.cache_need() != self.layers[src].mixer.cache_need():
                    raise ConfigError(f"run_order[{i}]: layer {entry.layer} cannot read the "
                                      f"cache of layer {src}: their cache needs differ")
                if src not in written:
                    raise ConfigError(f"run_order[{i}] reads the cache of layer {src} "
                                      f"before that layer has run")
                group, slot = owners[src]
                write = False
            elif entry.layer in owners:
                group, slot = owners[entry.layer]
                if entry.layer in written:
                    raise ConfigError(f"run_order[{i}] runs layer {entry.layer} a second "
                                      f"time and would write its cache twice; name "
                                      f"cache_of to read it instead")
                written.add(entry.layer)
            bindings.append(LayerBinding(group=group, slot=slot or 0, write=write,
                                         state_offset=state_offsets.get(entry.layer, 0),
                                         state_bytes=nbytes))
        specs = [CacheGroupSpec(need, tuple(members)) for need, members in groups]
        return specs, bindings, total_state

    # -- tensors ------------------------------------------------------------

    def _parts(self):
        """(path, part, layer index or None) for every part that has tensors."""
        yield "embedding", self.embedding, None
        yield "head", self.head, None
        yield "final_norm", self.final_norm, None
        for li, layer in enumerate(self.layers):
            for name, norm in layer.norms.items():
                yield f"layer.{name}", norm, li
            yield "layer.mixer", layer.mixer, li
            yield "layer.feed_forward", layer.feed_forward, li

    def tensor_requests(self) -> List[TensorRequest]:
        names = self.config.tensor_names
        out = []
        for path, part, li in self._parts():
            for decl in part.tensors():
                local = f"{path}.{decl.name}"
                if local not in names:
                    raise ConfigError(f"architecture {self.config.architecture!r} gives no "
                                      f"checkpoint name for {local!r}")
                ckpt = names[local].format(layer=li) if li is not None else names[local]
                key = local if li is None else f"{local}@{li}"
                out.append(TensorRequest(key, ckpt, decl))
        return out

    def bind(self, loaded: Dict[str, Optional[torch.Tensor]], dtype: torch.dtype,
             device: torch.device) -> None:
        self.dtype, self.device = dtype, device
        for path, part, li in self._parts():
            mine = {}
            for decl in part.tensors():
                key = f"{path}.{decl.name}" if li is None else f"{path}.{decl.name}@{li}"
                mine[decl.name] = loaded.get(key)
            part.bind(mine, dtype, device)
        if self.config.tie_word_embeddings:
            self.head.tie(self.embedding.table)

    @property
    def graph_safe(self) -> bool:
        return self._graph_flags()[0]

    @property
    def graph_safe_prompt_steps(self) -> bool:
        return self._graph_flags()[1]

    def _graph_flags(self):
        """(decode steps may be captured, steps with prompt portions may be captured): what
        the parts say about themselves, asked once."""
        flags = self.__dict__.get("_graph_flags_cache")
        if flags is None:
            def prompt_ok(part):
                flag = getattr(part, "graph_safe_prompt_steps", None)
                return getattr(part, "graph_safe", True) if flag is None else flag
            parts = [part for _, part, _ in self._parts()]
            flags = (all(getattr(part, "graph_safe", True) for part in parts),
                     all(prompt_ok(part) for part in parts))
            self._graph_flags_cache = flags
        return flags

    # -- one step -------------------------------------------------------------

    def forward(self, ctx) -> torch.Tensor:
        """Runs the step's tokens; returns fp32 logits [wanted rows, vocab]."""
        x = self.embedding.forward(ctx, ctx.token_ids)
        order = self.config.run_order
        for i, (entry, binding) in enumerate(zip(order, self.bindings)):
            # the norm that reads the rows after this layer, for the layer's last product
            nxt = self.layers[order[i + 1].layer] if i + 1 < len(order) else None
            entry_norm = getattr(nxt, "entry_norm", None)
            ctx.norm_after_layer = entry_norm() if entry_norm is not None else None
            self.layers[entry.layer].forward(ctx, x, binding)
        ctx.norm_after_layer = None
        if ctx.n_logit_rows == 0:
            return ctx.scratch("logits", (0, self.config.vocab_size), torch.float32)
        if ctx.host.all_single_token and ctx.n_logit_rows == ctx.n_tokens:
            # every request brings one token and wants its logits: the wanted rows are the
            # step's rows in order (a fact of the step's shape, so a captured step replays)
            rows = x
        else:
            rows = ctx.scratch("head.rows", (ctx.n_logit_rows, self.config.hidden_size),
                               torch.float32)
            ops.gather_rows(x, ctx.logit_rows, rows)
        h = self.final_norm.forward(ctx, rows)
        return self.head.forward(ctx, h)
