"""QLoRA: the frozen base matrices of every decoder layer are kept as 4-bit blocks and turned back into the compute
dtype only while their layer runs; the low-rank adapters beside them train in full precision.

``quantize_base_weights`` takes the attention, feed-forward and expert matrices of each layer out of the module's
parameters and stores them packed (``halo_b200.ops.nf4``). The layer's entry points (``forward``, and the two
halves the recomputation policies call on their own) are wrapped so that the matrices of the half that is about
to run appear as plain tensor attributes for the duration of the call and disappear again afterwards. With
per-layer recomputation the backward pass re-enters the layer, so at any moment only one layer's matrices exist in
the compute dtype: the resident cost of the base model is about 0.53 bytes per parameter (0.52 with nested maxima).

Everything that reads ``model.named_parameters()`` afterwards sees the adapters, norms, router and embeddings
only - which is what the optimizer, the gradient reduction and the adapter save need. Merging adapters into a
quantised base is refused: the merged matrix would be the rounded base plus the update, not the checkpoint's.
(The role of the reference's ``load_in_4bit`` path: bitsandbytes ``Linear4bit`` under PEFT,
halo/model_loading/dtype.py:114-119 and halo/model_loading/parallel/peft_setup.py.)"""

from __future__ import annotations

import contextlib

import torch

from halo_b200.ops.nf4 import Packed4bit, dequantize_4bit, quantize_4bit

# (owner path inside a decoder layer, attribute) per half of the layer
ATTENTION_WEIGHTS = (("self_attn", "qkv_proj"), ("self_attn", "o_proj"))
FEED_FORWARD_WEIGHTS = (("mlp", "gate_up_proj"), ("mlp", "down_proj"), ("mlp", "experts_gate_up"), ("mlp", "experts_down"),
                        ("mlp.shared_expert", "gate_up_proj"), ("mlp.shared_expert", "down_proj"))


class QuantizedLayerWeights:
    """The packed matrices of one decoder layer and the bookkeeping that shows them to the layer while it runs."""

    def __init__(self, layer, kind: str, nested: bool):
        self.layer = layer
        self.entries: dict[str, list[tuple[torch.nn.Module, str, Packed4bit]]] = {"attention": [], "feed_forward": []}
        self._depth = {"attention": 0, "feed_forward": 0}
        for half, wanted in (("attention", ATTENTION_WEIGHTS), ("feed_forward", FEED_FORWARD_WEIGHTS)):
            for path, attr in wanted:
                owner = layer
                for part in path.split("."):
                    owner = getattr(owner, part, None)
                    if owner is None:
                        break
                p = owner._parameters.get(attr) if owner is not None else None
                if p is None:
                    continue
                if p.requires_grad:
                    raise ValueError(f"{path}.{attr} is trainable: only frozen base weights are stored in 4 bits "
                                     f"(attach the adapters first)")
                self.entries[half].append((owner, attr, quantize_4bit(p.data, kind, nested)))
                del owner._parameters[attr]          # from here on the attribute exists only while the layer runs

    @contextlib.contextmanager
    def shown(self, *halves):
        fresh = [h for h in halves if self._depth[h] == 0]
        for h in halves:
            self._depth[h] += 1
        for h in fresh:
            for owner, attr, packed in self.entries[h]:
                setattr(owner, attr, dequantize_4bit(packed))
        try:
            yield
        finally:
            for h in halves:
                self._depth[h] -= 1
            for h in fresh:
                for owner, attr, _ in self.entries[h]:
                    delattr(owner, attr)

    def packed(self):
        return [(owner, attr, p) for half in self.entries.values() for owner, attr, p in half]

    @property
    def nbytes(self) -> int:
        return sum(p.nbytes for _, _, p in self.packed())


def _wrap(layer, store: QuantizedLayerWeights, name: str, halves: tuple):
    inner = getattr(layer, name)

    def entry(*args, **kw):
        with store.shown(*halves):
            return inner(*args, **kw)

    entry.__name__ = name
    object.__setattr__(layer, name, entry)


def decoder_layers(model):
    layers = list(model.layers)
    mtp = getattr(model, "mtp", None)
    if mtp is not None and getattr(mtp, "layer", None) is not None:
        layers.append(mtp.layer)
    return layers


def quantize_base_weights(model, kind: str = "nf4", nested: bool = False) -> dict:
    """Store every decoder layer's frozen matrices in 4 bits. Returns ``{"matrices", "parameters", "bytes"}``."""
    if getattr(model, "tensor_parallel", None) is not None or getattr(model, "expert_tensor_parallel", None) is not None:
        raise ValueError("4-bit base weights are stored whole per rank: tensor / expert-tensor parallel slices are not built for them")
    if getattr(model, "quantized_base", None) is not None:
        raise ValueError("the base weights of this model are already stored in 4 bits")
    stores, n_params = [], 0
    for layer in decoder_layers(model):
        store = QuantizedLayerWeights(layer, kind, nested)
        _wrap(layer, store, "forward", ("attention", "feed_forward"))
        _wrap(layer, store, "attention_half", ("attention",))
        _wrap(layer, store, "mlp_half", ("feed_forward",))
        layer.quantized_weights = store
        stores.append(store)
        n_params += sum(int(torch.tensor(p.shape).prod()) for _, _, p in store.packed())
    model.quantized_base = stores
    model.quantized_kind = kind
    return {"matrices": sum(len(s.packed()) for s in stores), "parameters": n_params, "bytes": sum(s.nbytes for s in stores)}


def is_quantized(model) -> bool:
    return getattr(model, "quantized_base", None) is not None


def dequantized_base_state(model) -> dict[str, torch.Tensor]:
    """Runtime parameter name -> the rounded base matrix in the compute dtype (for inspection and tests)."""
    names = {id(m): n for n, m in model.named_modules()}
    return {f"{names[id(owner)]}.{attr}": dequantize_4bit(p) for store in model.quantized_base for owner, attr, p in store.packed()}
