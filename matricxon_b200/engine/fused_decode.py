"""A decode step of the whole model as one persistent kernel (csrc/decode_fused.cu).

``FusedDecode.try_build`` reads the model's own description (``DecoderModel.describe``:
blocks as plain data) and answers with an object when every schedule entry is a pre-norm
block of LayerNorm, paged attention with a NeoX rotation over the whole head, and an MLP
with the tanh GELU, all of one geometry that the kernel takes; otherwise with None, and
the step runner keeps the part-by-part path. The parts know nothing of this file.

The reference runs a decode step as a sequence of module calls
(app/architectures/starcoder2.py:117-137); the arithmetic here is the same, the order of
memory traffic is not: the kernel's comment says how.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from matricxon_b200.ops.library import KernelLibraryError, check, library, register_signature

MAX_GROUPS = 4
MAX_ROWS = 16


class _Layer(ctypes.Structure):
    _fields_ = [(name, c_void_p) for name in (
        "ln1_w", "ln1_b", "ln2_w", "ln2_b", "qkv_w", "o_w", "fc_w", "proj_w", "qkv_b", "o_b", "fc_b",
        "proj_b", "inv_freq", "cache", "qkv_map", "o_map", "fc_map", "proj_map")] + [
        ("n_pages", c_longlong), ("ln1_eps", c_float), ("ln2_eps", c_float), ("scale_log2", c_float),
        ("window", c_int), ("group", c_int), ("writes_cache", c_int)]


class _Params(ctypes.Structure):
    _fields_ = [
        ("layers", c_void_p), ("token_ids", c_void_p), ("tok_seq", c_void_p), ("context_lens", c_void_p),
        ("slots", c_void_p * MAX_GROUPS), ("block_tables", c_void_p * MAX_GROUPS),
        ("bt_stride", c_int * MAX_GROUPS),
        ("embedding", c_void_p), ("final_w", c_void_p), ("final_b", c_void_p), ("head", c_void_p),
        ("head_map", c_void_p), ("x", c_void_p), ("xb", c_void_p), ("q", c_void_p), ("attn", c_void_p), ("mid", c_void_p), ("part_o", c_void_p),
        ("part_ml", c_void_p), ("stats", c_void_p), ("logits", c_void_p), ("barrier", c_void_p),
        ("status", c_void_p), ("final_eps", c_float),
        ("n_layers", c_int), ("rows", c_int), ("hidden", c_int), ("n_heads", c_int), ("n_kv_heads", c_int),
        ("head_dim", c_int), ("inter", c_int), ("vocab", c_int), ("page_size", c_int), ("n_splits", c_int),
        ("x_cols", c_int), ("xs_bytes", c_int), ("ring_slots", c_int), ("grid", c_int)]


register_signature("mx_decode_fused_sizes", [ctypes.POINTER(c_int), ctypes.POINTER(c_int)])
register_signature("mx_decode_fused_plan", [ctypes.POINTER(_Params)])
register_signature("mx_decode_fused", [ctypes.POINTER(_Params), c_void_p])
register_signature("mx_decode_fused_weight_map", [c_void_p, c_void_p, c_longlong, c_longlong, c_int])

MAP_BYTES = 128


class _TensorMaps:
    """Tensor maps over weight matrices, encoded on the host and kept in one device buffer."""

    def __init__(self) -> None:
        self._blobs: list[bytes] = []
        self.device_buffer: torch.Tensor | None = None

    def add(self, weight: torch.Tensor, box_rows: int) -> int:
        """Encodes the map of ``weight`` [rows, cols]; returns its index."""
        blob = ctypes.create_string_buffer(MAP_BYTES)
        check(library().mx_decode_fused_weight_map(blob, weight.data_ptr(), weight.shape[0], weight.shape[1],
                                                   box_rows), "fused decode tensor map")
        self._blobs.append(blob.raw)
        return len(self._blobs) - 1

    def upload(self, device: torch.device) -> None:
        raw = bytearray(b"".join(self._blobs))
        self.device_buffer = torch.frombuffer(raw, dtype=torch.uint8).to(device)
        if self.device_buffer.data_ptr() % 64 != 0:
            raise KernelLibraryError("tensor maps must start on a 64-byte boundary")

    def address(self, index: int) -> int:
        return self.device_buffer.data_ptr() + index * MAP_BYTES

LOG2E = 1.4426950408889634


def _ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


def _matrix_ok(weight: torch.Tensor, rows: int, cols: int) -> bool:
    return (weight.dtype == torch.bfloat16 and weight.is_cuda and weight.is_contiguous()
            and tuple(weight.shape) == (rows, cols) and weight.data_ptr() % 16 == 0)


def _vector_ok(vector: torch.Tensor | None, size: int) -> bool:
    return vector is None or (vector.dtype == torch.float32 and vector.is_contiguous()
                              and vector.numel() == size and vector.data_ptr() % 16 == 0)


class FusedDecode:
    """Holds the per-layer argument array and, per batch size, the buffers of a step."""

    def __init__(self, layers, geometry: dict, tensors: dict, device: torch.device, keep: list,
                 maps: _TensorMaps) -> None:
        self.maps = maps
        self.geometry = geometry
        self.tensors = tensors
        self.device = device
        self._keep = keep                                  # every tensor the device structures point into
        array = (_Layer * len(layers))(*layers)
        raw = bytes(array)
        self.layer_array = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(device)
        self.n_layers = len(layers)
        self._plans: dict[int, tuple] = {}

    # ------------------------------------------------------------------ construction
    @classmethod
    def try_build(cls, model, page_size: int) -> "FusedDecode | None":
        runtime = model.runtime
        if runtime.dtype != torch.bfloat16:
            return None
        description = model.describe()
        if description is None or not description["entries"]:
            return None
        sizes = (c_int(), c_int())
        library().mx_decode_fused_sizes(ctypes.byref(sizes[0]), ctypes.byref(sizes[1]))
        if sizes[0].value != ctypes.sizeof(_Layer) or sizes[1].value != ctypes.sizeof(_Params):
            raise KernelLibraryError("the fused decode kernel's argument blocks do not match this package")
        hidden = description["hidden_size"]
        vocab = description["vocab_size"]
        geometry = None
        layers, keep = [], []
        maps = _TensorMaps()
        map_index = []
        for entry in description["entries"]:
            block, binding = entry["block"], entry["binding"]
            if block["kind"] != "pre_norm_sequential":
                return None
            norm1, mixer, norm2, ffn = (block["mixer_norm"], block["mixer"], block["ffn_norm"],
                                        block["feed_forward"])
            if norm1["kind"] != "layernorm" or norm2["kind"] != "layernorm":
                return None
            if mixer["kind"] != "paged_attention" or ffn["kind"] != "mlp" or ffn["activation"] != "gelu_tanh":
                return None
            position = mixer["position"]
            heads, kv_heads, head_dim = mixer["num_heads"], mixer["num_kv_heads"], mixer["head_dim"]
            if position is None or position["kind"] != "rotary_neox" or position["rotary_dim"] != head_dim:
                return None
            if binding.kv is None or binding.group is None or binding.group >= MAX_GROUPS:
                return None
            inter = ffn["up_weight"].shape[0]
            here = (heads, kv_heads, head_dim, inter)
            if geometry is None:
                geometry = here
            elif geometry != here:
                return None                                # the kernel takes one geometry for all layers
            q_size = heads * head_dim
            ok = (_matrix_ok(mixer["qkv_weight"], q_size + 2 * kv_heads * head_dim, hidden)
                  and _matrix_ok(mixer["o_weight"], hidden, q_size)
                  and _matrix_ok(ffn["up_weight"], inter, hidden)
                  and _matrix_ok(ffn["down_weight"], hidden, inter)
                  and _vector_ok(mixer["qkv_bias"], q_size + 2 * kv_heads * head_dim)
                  and _vector_ok(mixer["o_bias"], hidden) and _vector_ok(ffn["up_bias"], inter)
                  and _vector_ok(ffn["down_bias"], hidden)
                  and _vector_ok(norm1["weight"], hidden) and _vector_ok(norm1["bias"], hidden)
                  and _vector_ok(norm2["weight"], hidden) and _vector_ok(norm2["bias"], hidden)
                  and _vector_ok(position["inv_freq"], head_dim // 2))
            cache = binding.kv
            if not ok or cache.dtype != torch.bfloat16 or not cache.is_contiguous():
                return None
            layer = _Layer(
                ln1_w=_ptr(norm1["weight"]), ln1_b=_ptr(norm1["bias"]), ln2_w=_ptr(norm2["weight"]),
                ln2_b=_ptr(norm2["bias"]), qkv_w=_ptr(mixer["qkv_weight"]), o_w=_ptr(mixer["o_weight"]),
                fc_w=_ptr(ffn["up_weight"]), proj_w=_ptr(ffn["down_weight"]), qkv_b=_ptr(mixer["qkv_bias"]),
                o_b=_ptr(mixer["o_bias"]), fc_b=_ptr(ffn["up_bias"]), proj_b=_ptr(ffn["down_bias"]),
                inv_freq=_ptr(position["inv_freq"]), cache=_ptr(cache), n_pages=cache.shape[0],
                ln1_eps=norm1["eps"], ln2_eps=norm2["eps"], scale_log2=mixer["scale"] * LOG2E,
                window=int(mixer["window"] or 0), group=int(binding.group),
                writes_cache=1 if binding.writes else 0)
            layers.append(layer)
            map_index.append((maps.add(mixer["qkv_weight"], 8), maps.add(mixer["o_weight"], 16),
                              maps.add(ffn["up_weight"], 16), maps.add(ffn["down_weight"], 16)))
            keep.extend([norm1, mixer, norm2, ffn, cache])
        final_norm = description["final_norm"]
        embedding, head = description["embedding"], description["head"]
        if final_norm["kind"] != "layernorm" or not _vector_ok(final_norm["weight"], hidden) \
                or not _vector_ok(final_norm["bias"], hidden):
            return None
        if not _matrix_ok(embedding, vocab, hidden) or not _matrix_ok(head, vocab, hidden):
            return None
        heads, kv_heads, head_dim, inter = geometry
        geometry = {"hidden": hidden, "vocab": vocab, "n_heads": heads, "n_kv_heads": kv_heads,
                    "head_dim": head_dim, "inter": inter, "page_size": page_size}
        tensors = {"embedding": embedding, "head": head, "final_w": final_norm["weight"],
                   "final_b": final_norm["bias"], "final_eps": final_norm["eps"]}
        head_index = maps.add(head, 16)
        maps.upload(runtime.device)
        for layer, (qkv, o, fc, proj) in zip(layers, map_index):
            layer.qkv_map, layer.o_map = maps.address(qkv), maps.address(o)
            layer.fc_map, layer.proj_map = maps.address(fc), maps.address(proj)
        tensors["head_map"] = maps.address(head_index)
        fused = cls(layers, geometry, tensors, runtime.device, keep, maps)
        probe = fused._blank_params(1)
        if library().mx_decode_fused_plan(ctypes.byref(probe)) != 0:
            return None                                    # a size the kernel refuses: the usual path runs
        return fused

    def _blank_params(self, rows: int) -> _Params:
        g, t = self.geometry, self.tensors
        return _Params(
            layers=self.layer_array.data_ptr(), embedding=_ptr(t["embedding"]), final_w=_ptr(t["final_w"]),
            final_b=_ptr(t["final_b"]), head=_ptr(t["head"]), head_map=t["head_map"], final_eps=t["final_eps"],
            n_layers=self.n_layers, rows=rows, hidden=g["hidden"], n_heads=g["n_heads"],
            n_kv_heads=g["n_kv_heads"], head_dim=g["head_dim"], inter=g["inter"], vocab=g["vocab"],
            page_size=g["page_size"], n_splits=1)

    def supports(self, rows: int) -> bool:
        return 1 <= rows <= MAX_ROWS

    # ------------------------------------------------------------------ one step
    def _plan(self, rows: int, max_kv_len: int):
        """Buffers and the fixed part of the argument block for steps of ``rows`` rows."""
        plan = self._plans.get(rows)
        if plan is not None:
            return plan
        g = self.geometry
        params = self._blank_params(rows)
        check(library().mx_decode_fused_plan(ctypes.byref(params)), "fused decode plan")
        grid = params.grid
        chunks = max(1, (max_kv_len + 31) // 32)
        n_splits = max(1, min(grid // max(rows * g["n_kv_heads"], 1), chunks))
        dev = self.device
        q_size = g["n_heads"] * g["head_dim"]
        buffers = {
            "x": torch.empty((rows, g["hidden"]), dtype=torch.float32, device=dev),
            "xb": torch.empty((rows, g["hidden"]), dtype=torch.bfloat16, device=dev),
            "q": torch.empty((rows, q_size), dtype=torch.bfloat16, device=dev),
            "attn": torch.empty((rows, q_size), dtype=torch.bfloat16, device=dev),
            "mid": torch.empty((rows, g["inter"]), dtype=torch.bfloat16, device=dev),
            "part_o": torch.empty((rows * g["n_heads"] * n_splits * g["head_dim"],), dtype=torch.float32, device=dev),
            "part_ml": torch.empty((rows * g["n_heads"] * n_splits * 2,), dtype=torch.float32, device=dev),
            "stats": torch.zeros((16 * ((grid + 31) // 32 * 32) * 4,), dtype=torch.float32, device=dev),
            "logits": torch.empty((rows, g["vocab"]), dtype=torch.float32, device=dev),
            "barrier": torch.zeros((4,), dtype=torch.int32, device=dev),
        }
        params.n_splits = n_splits
        for name in ("x", "xb", "q", "attn", "mid", "part_o", "part_ml", "stats", "logits", "barrier"):
            setattr(params, name, buffers[name].data_ptr())
        plan = (params, buffers)
        self._plans[rows] = plan
        return plan

    def forward(self, ctx) -> torch.Tensor:
        """Runs the step described by ``ctx`` (one token per row) and returns float32 logits
        [rows, vocab]; they live in this object's buffers until the next step of that size."""
        rows = ctx.n_tokens
        params, buffers = self._plan(rows, ctx.max_kv_len)
        params.token_ids = ctx.token_ids.data_ptr()
        params.tok_seq = ctx.tok_seq.data_ptr()
        params.context_lens = ctx.context_lens.data_ptr()
        params.status = ctx.status.data_ptr()
        if len(ctx.groups) > MAX_GROUPS:
            raise KernelLibraryError("fused decode takes at most four cache groups")
        for index, group in enumerate(ctx.groups):
            params.slots[index] = group.slots.data_ptr()
            params.block_tables[index] = group.block_tables.data_ptr()
            params.bt_stride[index] = group.block_tables.shape[1]
        stream = torch.cuda.current_stream().cuda_stream
        check(library().mx_decode_fused(ctypes.byref(params), stream), "fused decode")
        from matricxon_b200.ops import kernels
        kernels._launched()
        return buffers["logits"]
