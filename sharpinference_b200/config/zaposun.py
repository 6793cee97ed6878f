"""``ZaposunConfig``: the typed configuration of the Zaposun architecture.

A Zaposun ``config.json`` gives

* ``vocab``, ``width``, ``streams`` (residual streams per token), ``logit_scale``;
* ``norm``: ``eps`` and ``groups`` (every norm over the width is an RMS norm in that many equal parts);
* ``embedding.bigram``: ``buckets``, ``mul_prev``, ``mul_cur`` of the hashed pair table;
* ``layers``: a list of ``{"type", "mixer", "mlp"}``.  ``type`` is ``"wkv"`` (``mixer``: ``heads``, ``dim``; the inner
  size of the decay's two projections is the stored tensor's, or ``decay_rank`` where there is no file) or
  ``"parallel"`` (``mixer.left``: chunked attention with ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``,
  ``rot.dims`` / ``rot.base``, ``mask.size``; ``mixer.right``: a selective scan with ``inner``, ``state``,
  ``dt_rank``, ``conv``).  ``mlp`` is null or ``{"kind": "dense", "ff"}``.

No size stands in code; every layer may have sizes of its own.  Defaults for what a file may leave out:
``kv_heads`` = ``heads``, ``vdim`` = ``dim``, ``scale`` = ``dim^(-1/2)``, no ``rot`` = no rotation of q and k,
no ``mask`` = every earlier position, ``rot.base`` = 10000, ``streams`` = 1, ``norm.groups`` = 1,
``logit_scale`` = 1, ``rot.layout`` = ``"halves"`` (``"interleaved"`` pairs neighbours).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigReader
from .notedra import _merge


@dataclass(frozen=True)
class ZaposunAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int = 0
    rot_base: float = 10000.0
    rot_layout: str = "halves"
    chunk: int = 0               # positions of one chunk (0: every earlier position is visible)

    def to_dict(self) -> dict:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
               "rot": {"dims": self.rot_dims, "base": self.rot_base}}
        if self.rot_layout != "halves":
            out["rot"]["layout"] = self.rot_layout
        if self.chunk:
            out["mask"] = {"size": self.chunk}
        return out


@dataclass(frozen=True)
class ZaposunScan:
    inner: int
    state: int
    dt_rank: int
    conv: int

    def to_dict(self) -> dict:
        return {"inner": self.inner, "state": self.state, "dt_rank": self.dt_rank, "conv": self.conv}


@dataclass(frozen=True)
class ZaposunLayer:
    type: str                                   # "wkv" | "parallel"
    ff: int = 0                                 # width of the dense feed-forward (0: none)
    heads: int = 0                              # wkv
    dim: int = 0                                # wkv
    decay_rank: int = 0                         # wkv: inner size of the decay's two projections (0: as stored)
    left: Optional[ZaposunAttention] = None     # parallel
    right: Optional[ZaposunScan] = None         # parallel

    def to_dict(self) -> dict:
        if self.type == "wkv":
            mixer = {"heads": self.heads, "dim": self.dim}
            if self.decay_rank:
                mixer["decay_rank"] = self.decay_rank
        else:
            mixer = {"left": self.left.to_dict(), "right": self.right.to_dict()}
        return {"type": self.type, "mixer": mixer, "mlp": {"kind": "dense", "ff": self.ff} if self.ff else None}


@dataclass(frozen=True)
class ZaposunConfig:
    vocab: int
    width: int
    eps: float
    groups: int
    streams: int
    logit_scale: float
    buckets: int
    mul_prev: int
    mul_cur: int
    layers: Tuple[ZaposunLayer, ...]

    architecture = "Zaposun"

    @classmethod
    def from_dict(cls, obj: dict, where: str = "config.json") -> "ZaposunConfig":
        r = ConfigReader(obj, where)
        vocab, width = r.int("vocab"), r.int("width")
        streams, logit_scale = r.int("streams", 1), r.float("logit_scale", 1.0)
        eps = groups = buckets = mul_prev = mul_cur = None
        norm = r.object("norm")
        if norm is not None:
            nr = ConfigReader(norm, f"{where}[norm]")
            eps, groups = nr.float("eps"), nr.int("groups", 1)
            _merge(r, nr)
        emb = r.object("embedding")
        if emb is not None:
            er = ConfigReader(emb, f"{where}[embedding]")
            bigram = er.object("bigram")
            if bigram is not None:
                br = ConfigReader(bigram, f"{where}[embedding][bigram]")
                buckets, mul_prev, mul_cur = br.int("buckets"), br.int("mul_prev"), br.int("mul_cur")
                _merge(er, br)
            _merge(r, er)
        raw_layers = obj.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            r.problem("key 'layers': expected a non-empty list of layer descriptions")
            raw_layers = []
        layers = []
        for i, entry in enumerate(raw_layers):
            layer = _read_layer(entry, f"{where}[layers][{i}]", r)
            if layer is not None:
                layers.append(layer)
        if r.ok:
            r.require(vocab > 0 and width > 0, f"vocab ({vocab}) and width ({width}) must be positive")
            r.require(eps >= 0, f"norm.eps must not be negative, found {eps}")
            r.require(groups > 0 and width % groups == 0, f"norm.groups ({groups}) must divide the width ({width})")
            r.require(1 <= streams <= 8, f"streams must be 1 to 8, found {streams}")
            r.require(buckets > 0, f"embedding.bigram.buckets must be positive, found {buckets}")
        r.finish()
        return cls(vocab=vocab, width=width, eps=eps, groups=groups, streams=streams, logit_scale=logit_scale,
                   buckets=buckets, mul_prev=mul_prev, mul_cur=mul_cur, layers=tuple(layers))

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "streams": self.streams,
                "logit_scale": self.logit_scale, "norm": {"eps": self.eps, "groups": self.groups},
                "embedding": {"bigram": {"buckets": self.buckets, "mul_prev": self.mul_prev, "mul_cur": self.mul_cur}},
                "layers": [layer.to_dict() for layer in self.layers]}


def _read_layer(entry, where: str, top: ConfigReader) -> Optional[ZaposunLayer]:
    if not isinstance(entry, dict):
        top.problem(f"{where}: expected an object, found {type(entry).__name__}")
        return None
    r = ConfigReader(entry, where)
    kind, mixer = r.str("type"), r.object("mixer")
    ff = 0
    mlp = entry.get("mlp")
    if mlp is not None:
        if not isinstance(mlp, dict):
            r.problem(f"key 'mlp': expected an object or null, found {type(mlp).__name__}")
        else:
            mr = ConfigReader(mlp, f"{where}[mlp]")
            mkind, ff = mr.str("kind"), mr.int("ff")
            if mr.ok:
                mr.require(mkind == "dense", f"key 'kind': expected 'dense', found {mkind!r}")
                mr.require(ff > 0, f"ff must be positive, found {ff}")
            _merge(r, mr)
    layer = None
    if kind is not None and kind not in ("wkv", "parallel"):
        r.problem(f"key 'type': expected 'wkv' or 'parallel', found {kind!r}")
    elif kind == "wkv" and mixer is not None:
        m = ConfigReader(mixer, f"{where}[mixer]")
        heads, dim, rank = m.int("heads"), m.int("dim"), m.int("decay_rank", 0)
        if m.ok:
            m.require(heads > 0 and dim > 0 and rank >= 0, f"heads ({heads}) and dim ({dim}) must be positive")
        _merge(r, m)
        if r.ok:
            layer = ZaposunLayer("wkv", ff=ff, heads=heads, dim=dim, decay_rank=rank)
    elif kind == "parallel" and mixer is not None:
        m = ConfigReader(mixer, f"{where}[mixer]")
        left, right = m.object("left"), m.object("right")
        att = scan = None
        if left is not None:
            att = _read_attention(left, f"{where}[mixer][left]", m)
        if right is not None:
            sr = ConfigReader(right, f"{where}[mixer][right]")
            inner, state, dt_rank, conv = sr.int("inner"), sr.int("state"), sr.int("dt_rank"), sr.int("conv")
            if sr.ok:
                sr.require(min(inner, state, dt_rank, conv) > 0,
                           f"inner ({inner}), state ({state}), dt_rank ({dt_rank}) and conv ({conv}) must be positive")
                scan = ZaposunScan(inner, state, dt_rank, conv)
            _merge(m, sr)
        _merge(r, m)
        if r.ok and att is not None and scan is not None:
            layer = ZaposunLayer("parallel", ff=ff, left=att, right=scan)
    _merge(top, r)
    return layer if r.ok else None


def _read_attention(obj: dict, where: str, top: ConfigReader) -> Optional[ZaposunAttention]:
    m = ConfigReader(obj, where)
    heads, dim = m.int("heads"), m.int("dim")
    kv_heads, vdim, scale = m.int("kv_heads", heads), m.int("vdim", dim), m.float("scale", None)
    rot, mask = m.object("rot", None), m.object("mask", None)
    rot_dims, rot_base, layout, chunk = 0, 10000.0, "halves", 0
    if rot is not None:
        rr = ConfigReader(rot, f"{where}[rot]")
        rot_dims, rot_base, layout = rr.int("dims"), rr.float("base", 10000.0), rr.str("layout", "halves")
        _merge(m, rr)
    if mask is not None:
        mr = ConfigReader(mask, f"{where}[mask]")
        chunk = mr.int("size")
        _merge(m, mr)
    att = None
    if m.ok:
        m.require(heads > 0 and dim > 0 and vdim > 0, f"heads ({heads}), dim ({dim}) and vdim ({vdim}) must be positive")
        m.require(kv_heads > 0 and heads % kv_heads == 0, f"heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        m.require(dim % 2 == 0 and vdim % 2 == 0, f"dim ({dim}) and vdim ({vdim}) must be even")
        m.require(rot_dims % 2 == 0 and 0 <= rot_dims <= dim, f"rot.dims ({rot_dims}) must be even and at most dim ({dim})")
        m.require(layout in ("halves", "interleaved"), f"rot.layout must be 'halves' or 'interleaved', found {layout!r}")
        m.require(chunk >= 0, f"mask.size must not be negative, found {chunk}")
        if m.ok:
            att = ZaposunAttention(heads, kv_heads, dim, vdim, float(dim) ** -0.5 if scale is None else scale,
                                   rot_dims, rot_base, layout, chunk)
    _merge(top, m)
    return att
