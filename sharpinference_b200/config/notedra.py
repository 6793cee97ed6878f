"""``NotedraConfig``: the typed configuration of the Notedra architecture.

A Notedra ``config.json`` describes the model layer by layer:

* ``vocab``, ``width``, ``norm.eps``;
* ``layers``: a list of ``{"type", "mixer", "mlp"}``.  ``type`` is ``"mlstm"`` (``mixer``: ``heads``, ``dim``,
  ``vdim``, ``gate_cap``) or ``"attention"`` (``mixer``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``,
  ``rot.dims`` / ``rot.base``, ``mask.size``).  ``mlp`` is null, ``{"kind": "dense", "ff"}`` or
  ``{"kind": "moe", "expert.ff", "router.experts", "router.top", "router.scale"}``;
* ``loop``: ``{"start", "stop", "times"}``: layers ``start .. stop - 1`` run ``times`` times in a row with the
  same weights (null or absent: every layer runs once).

No size stands in code; every layer may have sizes of its own.  An attention layer without ``mask`` sees every
earlier position, one without ``rot`` is not rotated, ``scale`` defaults to ``dim^(-1/2)``, ``kv_heads`` to
``heads`` and ``vdim`` to ``dim``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigReader


@dataclass(frozen=True)
class NotedraMLP:
    kind: str                   # "dense" | "moe"
    ff: int                     # width of the dense network, or of one expert
    experts: int = 0
    top: int = 0
    route_scale: float = 1.0

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "expert": {"ff": self.ff},
                "router": {"experts": self.experts, "top": self.top, "scale": self.route_scale}}


@dataclass(frozen=True)
class NotedraLayer:
    type: str                   # "mlstm" | "attention"
    heads: int
    dim: int                    # key/query size of a head
    vdim: int                   # value size of a head
    mlp: Optional[NotedraMLP]
    gate_cap: float = 0.0       # mlstm
    kv_heads: int = 0           # attention
    scale: float = 0.0          # attention: factor on q . k
    rot_dims: int = 0           # attention: leading elements of a head that are rotated (0: none)
    rot_base: float = 10000.0
    window: int = 0             # attention: positions visible, the query's own included (0: all earlier ones)

    def to_dict(self) -> dict:
        if self.type == "mlstm":
            mixer = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "gate_cap": self.gate_cap}
        else:
            mixer = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                     "scale": self.scale}
            if self.rot_dims:
                mixer["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
            if self.window:
                mixer["mask"] = {"size": self.window}
        return {"type": self.type, "mixer": mixer, "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class NotedraConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[NotedraLayer, ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0         # 0: no loop

    architecture = "Notedra"

    def layer_runs(self):
        """The order in which layers run: ``(layer, pass or None, first of its pass)`` per run."""
        runs, i = [], 0
        n = len(self.layers)
        while i < n:
            if self.loop_times and i == self.loop_start:
                for t in range(self.loop_times):
                    for j in range(self.loop_start, self.loop_stop):
                        runs.append((j, t, j == self.loop_start))
                i = self.loop_stop
            else:
                runs.append((i, None, False))
                i += 1
        return runs

    # -- reading -----------------------------------------------------------------------
    @classmethod
    def from_dict(cls, obj: dict, where: str = "config.json") -> "NotedraConfig":
        r = ConfigReader(obj, where)
        vocab, width = r.int("vocab"), r.int("width")
        norm = r.object("norm")
        eps = ConfigReader(norm, f"{where}[norm]") if norm is not None else None
        eps_value = None
        if eps is not None:
            eps_value = eps.float("eps")
            _merge(r, eps)
        raw_layers = obj.get("layers")
        layers = []
        if not isinstance(raw_layers, list) or not raw_layers:
            r.problem("key 'layers': expected a non-empty list of layer descriptions")
            raw_layers = []
        for i, entry in enumerate(raw_layers):
            layer = _read_layer(entry, f"{where}[layers][{i}]", r)
            if layer is not None:
                layers.append(layer)
        start = stop = times = 0
        loop = r.object("loop", None)
        if loop is not None:
            lr = ConfigReader(loop, f"{where}[loop]")
            start, stop, times = lr.int("start"), lr.int("stop"), lr.int("times")
            _merge(r, lr)
            if None not in (start, stop, times):
                r.require(0 <= start < stop <= len(raw_layers),
                          f"loop: start {start} and stop {stop} must satisfy 0 <= start < stop <= layers ({len(raw_layers)})")
                r.require(times >= 1, f"loop: times must be at least 1, found {times}")
        if r.ok:
            r.require(vocab > 0 and width > 0, f"vocab ({vocab}) and width ({width}) must be positive")
            r.require(eps_value is not None and eps_value >= 0, f"norm.eps must be a non-negative number, found {eps_value}")
        r.finish()
        return cls(vocab=vocab, width=width, eps=eps_value, layers=tuple(layers), loop_start=start, loop_stop=stop,
                   loop_times=times)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "layers": [layer.to_dict() for layer in self.layers]}
        if self.loop_times:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return out


def _merge(into: ConfigReader, other: ConfigReader) -> None:
    """Carry a nested reader's problems into the file's one list, with the place they were found."""
    for text in other._problems:
        into.problem(f"{other._where}: {text}")


def _read_layer(entry, where: str, top: ConfigReader) -> Optional[NotedraLayer]:
    if not isinstance(entry, dict):
        top.problem(f"{where}: expected an object, found {type(entry).__name__}")
        return None
    r = ConfigReader(entry, where)
    kind = r.str("type")
    mixer = r.object("mixer")
    layer = None
    if kind is not None and kind not in ("mlstm", "attention"):
        r.problem(f"key 'type': expected 'mlstm' or 'attention', found {kind!r}")
    elif kind is not None and mixer is not None:
        m = ConfigReader(mixer, f"{where}[mixer]")
        heads, dim = m.int("heads"), m.int("dim")
        vdim = m.int("vdim", dim)
        fields = {}
        if kind == "mlstm":
            fields["gate_cap"] = m.float("gate_cap")
            if m.ok:
                m.require(fields["gate_cap"] > 0, f"gate_cap must be positive, found {fields['gate_cap']}")
        else:
            fields["kv_heads"] = m.int("kv_heads", heads)
            fields["scale"] = m.float("scale", None)
            rot, mask = m.object("rot", None), m.object("mask", None)
            if rot is not None:
                rr = ConfigReader(rot, f"{where}[mixer][rot]")
                fields["rot_dims"], fields["rot_base"] = rr.int("dims"), rr.float("base")
                _merge(m, rr)
            if mask is not None:
                mr = ConfigReader(mask, f"{where}[mixer][mask]")
                fields["window"] = mr.int("size")
                _merge(m, mr)
            if m.ok:
                if fields["scale"] is None:
                    fields["scale"] = float(dim) ** -0.5
                m.require(fields["kv_heads"] > 0 and heads % fields["kv_heads"] == 0,
                          f"heads ({heads}) must be a multiple of kv_heads ({fields['kv_heads']})")
                m.require(dim % 2 == 0, f"dim ({dim}) must be even")
                rd = fields.get("rot_dims", 0)
                m.require(rd % 2 == 0 and 0 <= rd <= dim, f"rot.dims ({rd}) must be even and at most dim ({dim})")
                m.require(fields.get("window", 0) >= 0, f"mask.size must not be negative, found {fields.get('window')}")
        if m.ok:
            m.require(heads > 0 and dim > 0 and vdim > 0, f"heads ({heads}), dim ({dim}) and vdim ({vdim}) must be positive")
        mlp = _read_mlp(entry.get("mlp"), f"{where}[mlp]", r)
        if m.ok:
            layer = NotedraLayer(type=kind, heads=heads, dim=dim, vdim=vdim, mlp=mlp, **fields)
        _merge(r, m)
    _merge(top, r)
    return layer if r.ok else None


def _read_mlp(entry, where: str, top: ConfigReader) -> Optional[NotedraMLP]:
    if entry is None:
        return None
    if not isinstance(entry, dict):
        top.problem(f"{where}: expected an object or null, found {type(entry).__name__}")
        return None
    r = ConfigReader(entry, where)
    kind = r.str("kind")
    mlp = None
    if kind == "dense":
        ff = r.int("ff")
        if r.ok:
            r.require(ff > 0, f"ff must be positive, found {ff}")
            mlp = NotedraMLP("dense", ff)
    elif kind == "moe":
        expert, router = r.object("expert"), r.object("router")
        if expert is not None and router is not None:
            er, rr = ConfigReader(expert, f"{where}[expert]"), ConfigReader(router, f"{where}[router]")
            ff, experts, top_k, scale = er.int("ff"), rr.int("experts"), rr.int("top"), rr.float("scale", 1.0)
            if er.ok and rr.ok:
                rr.require(ff > 0 and experts > 0 and 1 <= top_k <= experts,
                           f"ff ({ff}) and experts ({experts}) must be positive and 1 <= top ({top_k}) <= experts")
            _merge(r, er)
            _merge(r, rr)
            if r.ok:
                mlp = NotedraMLP("moe", ff, experts, top_k, scale)
    elif kind is not None:
        r.problem(f"key 'kind': expected 'dense' or 'moe', found {kind!r}")
    _merge(top, r)
    return mlp if r.ok else None
