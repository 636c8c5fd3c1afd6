"""NSW2 weight files and the GPT config JSON beside them: the data formats on the caller's side of the hot path.

``Module.Save`` / ``Module.Load`` (src/NeuralSharp/Layers/Module.cs:15,204-271): little-endian; u32 magic 0x3257534E
("NSW2"), i32 tensor count, then per tensor i32 rank, `rank` i32 dims and the raw float32 values; parameters in
``Parameters()`` order, then buffers.  ``GptConfig`` (samples/Shared/Gpt/CharGpt.cs:9-31) is a JSON record next to the
weights (same path, extension .json) with Vocabulary (one character per token), Context, Dim, Heads, Layers and
training bookkeeping.  ``CharGpt.Create`` (CharGpt.cs:107-124) fixes the tensor order: embedding [V, D]; per block
LayerNorm gamma/beta, fused QKV Linear [D, 3D] + bias, output Linear [D, D] + bias, LayerNorm gamma/beta, two
feed-forward Linears [D, 4D], [4D, D] with biases (TransformerEncoderLayer.Children, Layers/Attention.cs:214-217);
final LayerNorm; head Linear [D, V] + bias.  The positional table is not stored: it is recomputed
(PositionalEncoding, Layers/Attention.cs:236-246).
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np

from .gpt import GptConfig

FILE_MAGIC = 0x3257534E


class InvalidDataError(ValueError):
    """The reference's InvalidDataException."""


def read_nsw2(path: str) -> list:
    """All tensors of a weights file, in file order, as float32 arrays of their stored shapes."""
    with open(path, "rb") as f:
        data = f.read()
    if len(data) < 8 or struct.unpack_from("<I", data, 0)[0] != FILE_MAGIC:
        raise InvalidDataError(f"{path} is not a NeuralSharp weights file.")
    count = struct.unpack_from("<i", data, 4)[0]
    at, out = 8, []
    if count < 0:
        raise InvalidDataError(f"{path}: negative tensor count")
    for i in range(count):
        if at + 4 > len(data):
            raise InvalidDataError(f"{path}: truncated at tensor {i}")
        rank = struct.unpack_from("<i", data, at)[0]
        at += 4
        if rank < 0 or rank > 8 or at + 4 * rank > len(data):
            raise InvalidDataError(f"{path}: bad rank {rank} at tensor {i}")
        shape = struct.unpack_from(f"<{rank}i", data, at)
        at += 4 * rank
        if any(d < 0 for d in shape):
            raise InvalidDataError(f"{path}: bad shape {list(shape)} at tensor {i}")
        n = int(np.prod(shape, dtype=np.int64)) if rank else 1
        if at + 4 * n > len(data):
            raise InvalidDataError(f"{path}: truncated inside tensor {i} {list(shape)}")
        out.append(np.frombuffer(data, dtype="<f4", count=n, offset=at).astype(np.float32).reshape(shape))
        at += 4 * n
    return out


def write_nsw2(path: str, tensors) -> None:
    with open(path, "wb") as f:
        f.write(struct.pack("<Ii", FILE_MAGIC, len(tensors)))
        for t in tensors:
            a = np.asarray(t, dtype="<f4")          # keeps rank 0 (ascontiguousarray would make it rank 1)
            f.write(struct.pack(f"<i{a.ndim}i", a.ndim, *a.shape))
            f.write(a.tobytes(order="C"))


def config_path(weights_path: str) -> str:
    return os.path.splitext(weights_path)[0] + ".json"


def read_config(weights_path: str):
    """(GptConfig, vocabulary string) from the JSON record beside the weights; defaults as the record's (CharGpt.cs:9)."""
    with open(config_path(weights_path), "r", encoding="utf-8") as f:
        j = json.load(f)
    if not isinstance(j, dict) or "Vocabulary" not in j:
        raise InvalidDataError(f"Invalid model config {config_path(weights_path)}.")
    vocab = j["Vocabulary"]
    dim, heads = int(j.get("Dim", 96)), int(j.get("Heads", 4))
    cfg = GptConfig(vocab=len(vocab), dim=dim, heads=heads, layers=int(j.get("Layers", 3)), ff_dim=4 * dim, context=int(j.get("Context", 64)))
    return cfg, vocab


def write_config(weights_path: str, cfg: GptConfig, vocabulary: str) -> None:
    if len(vocabulary) != cfg.vocab or cfg.ff_dim != 4 * cfg.dim:
        raise ValueError("the config record describes vocab = len(Vocabulary) and ff_dim = 4 * Dim only")
    with open(config_path(weights_path), "w", encoding="utf-8") as f:
        json.dump({"Vocabulary": vocabulary, "Context": cfg.context, "Dim": cfg.dim, "Heads": cfg.heads, "Layers": cfg.layers,
                   "TrainedEpochs": 0, "ValidationLoss": None, "ValidationAccuracy": None, "TrainedAt": None, "Corpus": None}, f, indent=2)


def sinusoid_table(max_length: int, dim: int) -> np.ndarray:
    """PositionalEncoding's table (Layers/Attention.cs:236-246): angle = pos / 10000^(2*(i/2)/dim) in double,
    sin on even columns, cos on odd ones, rounded to float32."""
    pos = np.arange(max_length, dtype=np.float64)[:, None]
    i = np.arange(dim)
    angle = pos / np.power(10000.0, 2 * (i // 2) / float(dim))[None, :]
    return np.where(i % 2 == 0, np.sin(angle), np.cos(angle)).astype(np.float32)


def gpt_tensor_names(cfg: GptConfig) -> list:
    """(name, shape) of every tensor of a char-gpt weights file, in file order."""
    D, FF, V = cfg.dim, cfg.ff_dim, cfg.vocab
    names = [("tok", (V, D))]
    for i in range(cfg.layers):
        p = f"l{i}."
        names += [(p + "ln1_g", (D,)), (p + "ln1_b", (D,)), (p + "qkv_w", (D, 3 * D)), (p + "qkv_b", (3 * D,)), (p + "out_w", (D, D)),
                  (p + "out_b", (D,)), (p + "ln2_g", (D,)), (p + "ln2_b", (D,)), (p + "ff1_w", (D, FF)), (p + "ff1_b", (FF,)),
                  (p + "ff2_w", (FF, D)), (p + "ff2_b", (D,))]
    names += [("lnf_g", (D,)), ("lnf_b", (D,)), ("head_w", (D, V)), ("head_b", (V,))]
    return names


def load_char_gpt(weights_path: str):
    """(GptConfig, weight dict as the decoders of this package take it, vocabulary string).  Count and shapes must match
    the architecture the config describes, with the reference's messages (Module.cs:243-262)."""
    cfg, vocab = read_config(weights_path)
    tensors = read_nsw2(weights_path)
    names = gpt_tensor_names(cfg)
    if len(tensors) != len(names):
        raise InvalidDataError(f"The file has {len(tensors)} parameter tensors but the model has {len(names)}.")
    w = {}
    for (name, shape), t in zip(names, tensors):
        if tuple(t.shape) != tuple(shape):
            raise InvalidDataError(f"Shape mismatch: file has {list(t.shape)}, model has {list(shape)} ({name}).")
        w[name] = t
    w["pos"] = sinusoid_table(cfg.context, cfg.dim)
    return cfg, w, vocab


def save_char_gpt(weights_path: str, cfg: GptConfig, w: dict, vocabulary: str) -> None:
    write_nsw2(weights_path, [w[name] for name, _ in gpt_tensor_names(cfg)])
    write_config(weights_path, cfg, vocabulary)
