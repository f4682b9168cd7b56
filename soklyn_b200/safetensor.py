"""Checkpoint I/O in the reference's safetensors layout (src/io/safetensor.rs, src/io/save.rs).

File = 8-byte little-endian header length, JSON header, raw little-endian tensor bytes.
The writer reproduces the reference's bytes: the header is serde_json's pretty form of a map
whose keys come out sorted (its `Map` is a BTreeMap: `__metadata__` first, then the tensor
names; inside a tensor entry `data_offsets`, `dtype`, `shape`), padded with spaces to a
multiple of 8 bytes; tensor data follow in the order the tensors were passed.
Tensor names are `layer{N}.{w,b,norm_w,norm_b}` in the block's precision and, for training
blocks, `dv_*`, `dm_*` moments and (16-bit blocks) `master_*` copies in F32 (save.rs:227-346).
"""
from __future__ import annotations

import json
import os
import struct
import tempfile
from typing import Dict, List, Optional

import numpy as np

from . import log
from .function import Precision

_DTYPE = {Precision.FP32: ("F32", np.float32), Precision.FP16: ("F16", np.float16)}
_F32_ONLY = {"master_w", "master_b", "master_norm_w", "master_norm_b", "dv_w", "dv_b", "dm_w", "dm_b",
             "dv_norm_w", "dv_norm_b", "dm_norm_w", "dm_norm_b"}
_PARAMS = _F32_ONLY | {"w", "b", "norm_w", "norm_b"}


class SerdeError(log.Error):
    """JSON / format errors of a checkpoint file (Error::SerdeJSON, UnrecognizedTensorKey, ...)."""


class SafetensorWriter:
    """src/io/safetensor.rs:23-203"""

    def __init__(self):
        self.descriptors: List[dict] = []      # {name, shape, data(bytes), precision}
        self.metadata: Dict[str, str] = {}

    def pass_(self, name: str, shape, data: bytes, precision: Precision):
        self.descriptors.append({"name": name, "shape": [int(s) for s in shape], "data": bytes(data), "precision": precision})

    def pass_metadata(self, key: str, value: str):
        self.metadata[str(key)] = str(value)

    def header_bytes(self) -> bytes:
        header = {}
        if self.metadata:
            header["__metadata__"] = dict(self.metadata)
        off = 0
        for d in self.descriptors:
            end = off + len(d["data"])
            header[d["name"]] = {"dtype": _DTYPE[d["precision"]][0], "shape": d["shape"], "data_offsets": [off, end]}
            off = end
        text = json.dumps(header, indent=2, sort_keys=True, ensure_ascii=False).encode("utf-8")
        if len(text) % 8:
            text += b" " * (8 - len(text) % 8)
        return text

    def write(self, f):
        head = self.header_bytes()
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for d in self.descriptors:
            f.write(d["data"])
        f.flush()

    @staticmethod
    def read(f) -> "SafetensorWriter":
        raw = f.read(8)
        if len(raw) != 8:
            raise SerdeError("unexpected end of file in the header length")
        (n,) = struct.unpack("<Q", raw)
        head = f.read(n)
        if len(head) != n:
            raise SerdeError("unexpected end of file in the header")
        try:
            table = json.loads(head.decode("utf-8"))
        except ValueError as e:
            raise SerdeError(f"JSON error: {e}")
        w = SafetensorWriter()
        base = 8 + n
        for key, val in table.items():
            if key == "__metadata__":
                for mk, mv in (val or {}).items():
                    w.metadata[mk] = mv if isinstance(mv, str) else json.dumps(mv)
                continue
            dtype = val["dtype"]
            if dtype not in ("F32", "F16"):
                raise SerdeError(f"Tensor '{key}' has unrecognised dtype '{dtype}'.")
            a, b = val["data_offsets"]
            f.seek(base + a)
            data = f.read(b - a)
            if len(data) != b - a:
                raise SerdeError(f"unexpected end of file in tensor '{key}'")
            w.descriptors.append({"name": key, "shape": list(val["shape"]), "data": data,
                                  "precision": Precision.FP16 if dtype == "F16" else Precision.FP32})
        return w


class SafetensorFile:
    """src/io/save.rs:118-576"""

    def __init__(self):
        self.writer = SafetensorWriter()

    # ---- saving ----
    @staticmethod
    def from_ffn(context, network) -> "SafetensorFile":
        return SafetensorFile.from_blocks(context, network.get_layers())

    @staticmethod
    def from_blocks(context, blocks) -> "SafetensorFile":
        f = SafetensorFile()
        f.pass_blocks(context, blocks)
        return f

    def pass_blocks(self, context, blocks):
        for i, layer in enumerate(blocks):
            self.pass_layer(context, layer, i + 1)

    def pass_metadata(self, key, value):
        self.writer.pass_metadata(str(key), str(value))

    def get_metadata(self) -> Dict[str, str]:
        return self.writer.metadata

    def pass_layer(self, context, layer, layer_num: int):
        if layer.precision not in _DTYPE:
            raise log.UnsupportedTypeCast(layer.precision, "safetensors F32/F16")
        np_t = _DTYPE[layer.precision][1]
        k, n = layer.get_weights().rows(), layer.get_weights().cols()
        put = lambda suffix, shape, t, prec, dt: self.writer.pass_(
            f"layer{layer_num}.{suffix}", shape, np.ascontiguousarray(t.download(context), dtype=dt).tobytes(), prec)
        put("w", [k, n], layer.get_weights(), layer.precision, np_t)
        put("b", [n], layer.get_biases(), layer.precision, np_t)
        put("norm_w", [n], layer.get_norm_weights(), layer.precision, np_t)
        put("norm_b", [n], layer.get_norm_biases(), layer.precision, np_t)
        if not layer.is_training_mode():
            return
        f32 = Precision.FP32
        put("dv_w", [k, n], layer.get_dv_weights(), f32, np.float32)
        put("dv_b", [n], layer.get_dv_biases(), f32, np.float32)
        put("dm_w", [k, n], layer.get_dm_weights(), f32, np.float32)
        put("dm_b", [n], layer.get_dm_biases(), f32, np.float32)
        put("dv_norm_w", [n], layer.get_dv_norm_weights(), f32, np.float32)
        put("dv_norm_b", [n], layer.get_dv_norm_biases(), f32, np.float32)
        put("dm_norm_w", [n], layer.get_dm_norm_weights(), f32, np.float32)
        put("dm_norm_b", [n], layer.get_dm_norm_biases(), f32, np.float32)
        for suffix, t in (("master_w", layer.get_master_weights()), ("master_b", layer.get_master_biases()),
                          ("master_norm_w", layer.get_master_norm_weights()), ("master_norm_b", layer.get_master_norm_biases())):
            if t is not None:
                put(suffix, [t.rows(), t.cols()], t, f32, np.float32)

    def save(self, path: str):
        """Atomic: write a temporary file in the target directory, then rename (save.rs:365-375)."""
        directory = os.path.dirname(os.path.abspath(path)) or "."
        fd, tmp = tempfile.mkstemp(dir=directory)
        try:
            with os.fdopen(fd, "wb") as f:
                self.writer.write(f)
            os.replace(tmp, path)
        except BaseException:
            if os.path.exists(tmp):
                os.unlink(tmp)
            raise

    # ---- loading ----
    @staticmethod
    def read(path: str) -> "SafetensorFile":
        f = SafetensorFile()
        with open(path, "rb") as fh:
            f.writer = SafetensorWriter.read(fh)
        return f

    def layer_arrays(self, precision: Precision) -> Dict[int, Dict[str, np.ndarray]]:
        """{layer index: {param suffix: flat numpy array}} after the checks of save.rs:416-470."""
        layers: Dict[int, Dict[str, np.ndarray]] = {}
        for d in self.writer.descriptors:
            name = d["name"]
            if not name.startswith("layer"):
                continue
            rest = name[len("layer"):]
            if "." not in rest:
                raise SerdeError(f"Invalid tensor name format '{name}': missing '.' separator.")
            idx_s, param = rest.split(".", 1)
            if not idx_s.isdigit():
                raise SerdeError(f"Invalid tensor name format '{name}': invalid layer index number.")
            if param not in _PARAMS:
                raise SerdeError(f"Invalid tensor name format '{name}': unrecognized parameter type.")
            if param in _F32_ONLY and d["precision"] == Precision.FP16:
                raise SerdeError(f"Layer {idx_s}: '{param}' must be FP32 but safetensor file contains FP16.")
            want = Precision.FP32 if param in _F32_ONLY else precision
            if param not in _F32_ONLY and d["precision"] != want:
                raise SerdeError(f"Layer {idx_s}: '{param}' is stored as {d['precision'].name}, the blocks are {want.name}.")
            arr = np.frombuffer(d["data"], dtype=_DTYPE[d["precision"]][1]).copy()
            entry = layers.setdefault(int(idx_s), {})
            entry[param] = arr
            if param == "w":
                entry["_shape"] = tuple(d["shape"])
        return layers

    def into_blocks(self, context, is_training: bool, max_batch_size: int, precision: Precision = Precision.FP32):
        """Rebuild the blocks; configuration (normalisation, activation, ...) is not part of the
        file and comes back as Disabled / Identity, as in the reference (save.rs:567-572)."""
        from .context import LayerInitConfig
        from .core import Tensor
        from .mlp import DenseBlock, ParamState
        layers = self.layer_arrays(precision)
        if not layers or max(layers) == 0:
            raise SerdeError("No network layers were found in safetensor file.")
        blocks = []
        for idx in range(1, max(layers) + 1):
            if idx not in layers:
                raise SerdeError(f"Layer {idx} is completely missing from the safetensor file.")
            e = layers[idx]
            if "w" not in e:
                raise SerdeError(f"Weights for layer {idx} is completely missing from the safetensor file.")
            if "b" not in e:
                raise SerdeError(f"Biases for layer {idx} is completely missing from the safetensor file.")
            k, n = e["_shape"]
            t = lambda key, shape, prec: Tensor.from_cpu_vector(context, e[key], shape, prec)
            topt = lambda key, shape: (t(key, shape, Precision.FP32) if key in e else None)
            tdef = lambda key, shape: (t(key, shape, precision) if key in e else Tensor.zeros(context, shape, precision))
            mom = lambda key, shape: (topt(key, shape) if is_training else None)
            lin = ParamState(t("w", (k, n), precision), t("b", (1, n), precision), topt("master_w", (k, n)),
                             topt("master_b", (1, n)), mom("dv_w", (k, n)), mom("dv_b", (1, n)), mom("dm_w", (k, n)),
                             mom("dm_b", (1, n)))
            nrm = ParamState(tdef("norm_w", (1, n)), tdef("norm_b", (1, n)), topt("master_norm_w", (1, n)),
                             topt("master_norm_b", (1, n)), mom("dv_norm_w", (1, n)), mom("dv_norm_b", (1, n)),
                             mom("dm_norm_w", (1, n)), mom("dm_norm_b", (1, n)))
            blocks.append(DenseBlock.from_tensors(context, is_training, lin, nrm, max_batch_size, LayerInitConfig(), precision))
        return blocks
