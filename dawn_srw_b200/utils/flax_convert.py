"""Flax msgpack checkpoints <-> torch state dicts, without JAX.

The reference saves ``flax.serialization.to_bytes`` blobs (scripts/train_jax.py:
1096-1154).  That format is msgpack in which every array is an ExtType(1) whose
payload is itself msgpack ``(shape, dtype_name, raw_bytes)``; numpy scalars use
ExtType(3).  Only ``msgpack`` and ``numpy`` are needed to read or write it.

Name mapping for the SRW models (the reference ships a converter only for its
older model families, scripts/convert_flax_to_pt.py:82-139):

    token_emb/embedding            -> token_emb.weight
    pos_emb/embedding              -> pos_emb.weight
    neuron_pool/<name>             -> neuron_pool.<name>
    router/<lin>/kernel [in,out]   -> router.<lin>.weight [out,in]   (transposed)
    router/<lin>/bias              -> router.<lin>.bias
    block_<i>/norm{1,2}/scale|bias -> layers.<i>.norm{1,2}.weight|bias
    block_<i>/attn/expand_O/kernel -> layers.<i>.attn.expand_O.weight (transposed)
    norm/scale|bias                -> norm.weight|bias

Leading singleton axes left by device-replicated checkpoints are squeezed
(reference: models/dawn_spatial_v41_exp.py:1700-1710).
"""
from __future__ import annotations

import re
from typing import Any, Dict

import msgpack
import numpy as np
import torch

_EXT_NDARRAY, _EXT_NPSCALAR = 1, 3


def _ext_hook(code, data):
    if code == _EXT_NDARRAY:
        shape, dtype, buf = msgpack.unpackb(data, raw=False)
        return np.frombuffer(buf, dtype=np.dtype(dtype)).reshape(shape).copy()
    if code == _EXT_NPSCALAR:
        shape, dtype, buf = msgpack.unpackb(data, raw=False)
        return np.frombuffer(buf, dtype=np.dtype(dtype)).reshape(shape)[()]
    return msgpack.ExtType(code, data)


def _default(obj):
    if isinstance(obj, np.ndarray):
        payload = msgpack.packb((list(obj.shape), obj.dtype.name, obj.tobytes()), use_bin_type=True)
        return msgpack.ExtType(_EXT_NDARRAY, payload)
    if isinstance(obj, np.generic):
        a = np.asarray(obj)
        payload = msgpack.packb(([], a.dtype.name, a.tobytes()), use_bin_type=True)
        return msgpack.ExtType(_EXT_NPSCALAR, payload)
    raise TypeError(f"cannot serialise {type(obj)}")


def msgpack_restore(blob: bytes) -> Any:
    return msgpack.unpackb(blob, ext_hook=_ext_hook, raw=False, strict_map_key=False)


def msgpack_serialize(tree: Any) -> bytes:
    return msgpack.packb(tree, default=_default, use_bin_type=True)


def _squeeze(a: np.ndarray) -> np.ndarray:
    while a.ndim >= 2 and a.shape[0] == 1:
        a = a[0]
    return a


def flatten_tree(tree: Dict, prefix: str = "") -> Dict[str, np.ndarray]:
    out = {}
    for k, v in tree.items():
        key = f"{prefix}/{k}" if prefix else str(k)
        if isinstance(v, dict):
            out.update(flatten_tree(v, key))
        else:
            out[key] = v
    return out


def flax_name_to_torch(name: str):
    """-> (torch_name, transpose?)"""
    parts = name.split("/")
    m = re.fullmatch(r"block_(\d+)", parts[0])
    if m:
        parts[0] = f"layers.{m.group(1)}"
    leaf = parts[-1]
    transpose = False
    if leaf == "embedding":
        parts[-1] = "weight"
    elif leaf == "kernel":
        parts[-1] = "weight"
        transpose = True
    elif leaf == "scale" and any("norm" in p for p in parts[:-1]):
        parts[-1] = "weight"
    return ".".join(parts), transpose


def torch_name_to_flax(name: str, is_norm_weight: bool, is_dense_weight: bool, is_embedding: bool):
    parts = name.split(".")
    if parts[0] == "layers":
        parts = [f"block_{parts[1]}"] + parts[2:]
    if parts[-1] == "weight":
        parts[-1] = "embedding" if is_embedding else ("scale" if is_norm_weight else "kernel")
    return "/".join(parts), is_dense_weight


def flax_params_to_state_dict(params: Dict) -> Dict[str, torch.Tensor]:
    sd = {}
    for name, arr in flatten_tree(params).items():
        tname, tr = flax_name_to_torch(name)
        a = _squeeze(np.asarray(arr))
        if tr and a.ndim == 2:
            a = a.T
        sd[tname] = torch.from_numpy(np.ascontiguousarray(a))
    return sd


def state_dict_to_flax_params(sd: Dict[str, torch.Tensor]) -> Dict:
    tree: Dict = {}
    for name, t in sd.items():
        leaf_owner = name.rsplit(".", 1)[0]
        is_emb = leaf_owner in ("token_emb", "pos_emb")
        is_norm = "norm" in leaf_owner.split(".")[-1]
        is_dense = name.endswith(".weight") and not is_emb and not is_norm
        fname, tr = torch_name_to_flax(name, is_norm, is_dense, is_emb)
        a = t.detach().cpu().float().numpy()
        if tr and a.ndim == 2:
            a = a.T
        node = tree
        keys = fname.split("/")
        for k in keys[:-1]:
            node = node.setdefault(k, {})
        node[keys[-1]] = np.ascontiguousarray(a)
    return tree


# ---------------------------------------------------------------------------
# Optimizer state.  The reference's optimizer is an optax chain
#   clip_by_global_norm, scale_by_adam, add_decayed_weights (base mask),
#   add_decayed_weights (pool mask), scale_by_learning_rate(schedule)
# optionally wrapped in optax.MultiSteps (scripts/train_jax.py:2083-2120), and
# ``flax.serialization`` writes its state as nested dicts: a tuple becomes
# {"0": .., "1": ..}, a NamedTuple a dict of its fields, an empty state {}:
#   chain  = {"0": {}, "1": {"count", "mu": <param tree>, "nu": <param tree>},
#             "2": {"inner_state": {}}, "3": {"inner_state": {}}, "4": {"count"}}
#   wrapped = {"mini_step", "gradient_step", "inner_opt_state": chain,
#              "acc_grads": <param tree>, "skip_state": {}}
# The moments map onto DawnAdamW's exp_avg / exp_avg_sq (same names and
# transposes as the parameters), ``count`` onto its step counter, ``mini_step``
# and ``acc_grads`` onto the gradient-accumulation window.

def _scalar(x, default=0) -> int:
    if x is None:
        return default
    return int(np.asarray(x).reshape(-1)[0])


def optax_state_to_torch(opt_state: Dict) -> Dict[str, Any]:
    """Reference ``opt_state`` tree -> ``DawnAdamW.load_state_dict`` input."""
    wrapped = isinstance(opt_state, dict) and "inner_opt_state" in opt_state
    chain = opt_state["inner_opt_state"] if wrapped else opt_state
    adam = None
    for key in sorted(chain, key=str):
        node = chain[key]
        if isinstance(node, dict) and "mu" in node and "nu" in node:
            adam = node
            break
    if adam is None:
        raise ValueError("no scale_by_adam state (mu / nu) in the optimizer state")
    out: Dict[str, Any] = {
        "count": _scalar(adam.get("count")),
        "micro": _scalar(opt_state.get("mini_step")) if wrapped else 0,
        "exp_avg": flax_params_to_state_dict(adam["mu"]),
        "exp_avg_sq": flax_params_to_state_dict(adam["nu"]),
        "acc": None,
    }
    if wrapped and out["micro"] > 0 and opt_state.get("acc_grads"):
        # optax keeps the running MEAN of the window's gradients; DawnAdamW keeps their sum
        acc = flax_params_to_state_dict(opt_state["acc_grads"])
        out["acc"] = {k: v * float(out["micro"]) for k, v in acc.items()}
    return out


def torch_opt_state_to_optax(sd: Dict[str, Any], accumulation_steps: int = 1) -> Dict:
    """``DawnAdamW.state_dict()`` -> the reference's ``opt_state`` tree."""
    count = np.asarray(int(sd["count"]), dtype=np.int32)
    chain = {"0": {},
             "1": {"count": count, "mu": state_dict_to_flax_params(sd["exp_avg"]),
                   "nu": state_dict_to_flax_params(sd["exp_avg_sq"])},
             "2": {"inner_state": {}}, "3": {"inner_state": {}},
             "4": {"count": count}}
    if accumulation_steps <= 1:
        return chain
    micro = int(sd.get("micro", 0))
    acc = sd.get("acc")
    if acc is None or micro == 0:
        acc_tree = state_dict_to_flax_params({k: torch.zeros_like(v) for k, v in sd["exp_avg"].items()})
    else:
        acc_tree = state_dict_to_flax_params({k: v / float(micro) for k, v in acc.items()})
    return {"mini_step": np.asarray(micro, dtype=np.int32), "gradient_step": count,
            "inner_opt_state": chain, "acc_grads": acc_tree, "skip_state": {}}


def load_flax_checkpoint(path: str) -> Dict[str, Any]:
    """Read a reference ``.flax`` file.  Returns a dict with ``state_dict``
    (torch names), ``opt_state`` (``DawnAdamW.load_state_dict`` layout, or None
    when the file carries no optimizer state) plus the scalar fields (epoch,
    step, config, ...)."""
    with open(path, "rb") as f:
        raw = msgpack_restore(f.read())
    params = raw.get("params", raw)
    out = {k: v for k, v in raw.items() if k not in ("params", "opt_state")}
    out["state_dict"] = flax_params_to_state_dict(params)
    out["opt_state"] = None
    if isinstance(raw.get("opt_state"), dict) and raw["opt_state"]:
        out["opt_state"] = optax_state_to_torch(raw["opt_state"])
    return out


def save_flax_checkpoint(path: str, state_dict: Dict[str, torch.Tensor], opt_state=None,
                         accumulation_steps: int = 1, **fields) -> None:
    """Write a ``.flax`` file the reference can load.  ``opt_state`` is a
    ``DawnAdamW.state_dict()``; without it the field is an empty dict."""
    tree = {"params": state_dict_to_flax_params(state_dict),
            "opt_state": {} if opt_state is None else torch_opt_state_to_optax(opt_state, accumulation_steps),
            **fields}
    with open(path, "wb") as f:
        f.write(msgpack_serialize(tree))
