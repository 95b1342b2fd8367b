"""MAL (Model Architecture Language): the architecture config DSL.

A hand-written tokenizer + recursive-descent parser for the MAL grammar, the
resolved `ModelDef` dataclass tree, its serde-compatible JSON form, the exact
parameter-count estimator and the embedded presets.

Parity: grammar `summa-mal/src/mal.pest`, AST + defaults + estimator
`summa-mal/src/lib.rs:100-700`, entry points `parse_mal` / `parse_mal_full` /
`parse_mal_file` / `get_builtin_model` / `list_wellknown_models`
(`summa-mal/src/lib.rs:855,889,1504,1519,1541`).

The JSON form follows serde's externally-tagged enum encoding, e.g.
`{"Rope": {"theta": 10000.0, "scaling": null}}`, `"RmsNorm"`, `"SwiGLU"`, so a
`config.json` written by either implementation loads in the other.
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass, field
from typing import Dict, List, Optional

__all__ = [
    "MalError", "PositionEncoding", "AttentionDef", "SsmDef", "MoeDef", "FfnDef",
    "ReserveExpertsDef", "MemoryTierDef", "MemoryDef", "NormConfig", "BlockDef",
    "EmbeddingsConfig", "OutputConfig", "ModelDef", "MalFile", "parse_mal",
    "parse_mal_full", "parse_mal_file", "get_builtin_model",
    "list_wellknown_models", "load_model_def",
]


class MalError(ValueError):
    """Raised for syntax errors, duplicate names and unresolved references."""


# --------------------------------------------------------------------------
# AST
# --------------------------------------------------------------------------

@dataclass
class PositionEncoding:
    kind: str = "rope"              # rope | alibi | learned | none
    theta: float = 10000.0
    scaling: Optional[float] = None
    learned_slopes: bool = False
    max_positions: int = 0

    def to_json(self):
        if self.kind == "rope":
            return {"Rope": {"theta": float(self.theta), "scaling": self.scaling}}
        if self.kind == "alibi":
            return {"Alibi": {"learned_slopes": self.learned_slopes}}
        if self.kind == "learned":
            return {"Learned": {"max_positions": self.max_positions}}
        return "None"

    @staticmethod
    def from_json(v) -> "PositionEncoding":
        if v == "None" or v is None:
            return PositionEncoding(kind="none")
        if isinstance(v, dict) and len(v) == 1:
            (tag, body), = v.items()
            if tag == "Rope":
                return PositionEncoding("rope", float(body["theta"]), body.get("scaling"))
            if tag == "Alibi":
                return PositionEncoding("alibi", learned_slopes=bool(body["learned_slopes"]))
            if tag == "Learned":
                return PositionEncoding("learned", max_positions=int(body["max_positions"]))
        raise MalError(f"unknown position encoding {v!r}")


@dataclass
class AttentionDef:
    name: str = "default"
    num_heads: Optional[int] = None
    num_kv_heads: Optional[int] = None
    head_dim: Optional[int] = None
    dropout: float = 0.0
    bias: bool = False
    position_encoding: PositionEncoding = field(default_factory=PositionEncoding)
    window_size: Optional[int] = None
    causal: bool = True
    qk_norm: bool = False

    def to_json(self):
        return {
            "name": self.name, "num_heads": self.num_heads,
            "num_kv_heads": self.num_kv_heads, "head_dim": self.head_dim,
            "dropout": float(self.dropout), "bias": self.bias,
            "position_encoding": self.position_encoding.to_json(),
            "window_size": self.window_size, "causal": self.causal,
            "qk_norm": self.qk_norm,
        }

    @staticmethod
    def from_json(d) -> "AttentionDef":
        return AttentionDef(
            name=d["name"], num_heads=d.get("num_heads"),
            num_kv_heads=d.get("num_kv_heads"), head_dim=d.get("head_dim"),
            dropout=float(d["dropout"]), bias=bool(d["bias"]),
            position_encoding=PositionEncoding.from_json(d["position_encoding"]),
            window_size=d.get("window_size"), causal=bool(d["causal"]),
            qk_norm=bool(d.get("qk_norm", False)))


@dataclass
class SsmDef:
    name: str = "default"
    state_dim: int = 16
    conv_kernel: int = 4
    expand: int = 2
    dt_rank: Optional[int] = None

    def to_json(self):
        return {"name": self.name, "state_dim": self.state_dim,
                "conv_kernel": self.conv_kernel, "expand": self.expand,
                "dt_rank": self.dt_rank}

    @staticmethod
    def from_json(d) -> "SsmDef":
        return SsmDef(d["name"], int(d["state_dim"]), int(d["conv_kernel"]),
                      int(d["expand"]), d.get("dt_rank"))


@dataclass
class MoeDef:
    experts: int = 0
    top_k: int = 0
    shared_experts: int = 0
    load_balance_loss_weight: float = 0.0
    router_z_loss_weight: float = 0.0

    def to_json(self):
        return {"experts": self.experts, "top_k": self.top_k,
                "shared_experts": self.shared_experts,
                "load_balance_loss_weight": float(self.load_balance_loss_weight),
                "router_z_loss_weight": float(self.router_z_loss_weight)}

    @staticmethod
    def from_json(d) -> "MoeDef":
        return MoeDef(int(d["experts"]), int(d["top_k"]),
                      int(d.get("shared_experts", 0)),
                      float(d.get("load_balance_loss_weight", 0.0)),
                      float(d.get("router_z_loss_weight", 0.0)))


_ACT_TO_JSON = {"swiglu": "SwiGLU", "gelu": "GELU", "silu": "SiLU", "relu": "ReLU",
                "gelu_new": "GELUNew", "gelu_tanh": "GELUTanh"}
_ACT_FROM_JSON = {v: k for k, v in _ACT_TO_JSON.items()}


@dataclass
class FfnDef:
    name: str = "default"
    hidden_dim: Optional[int] = None
    activation: str = "swiglu"
    bias: bool = False
    dropout: float = 0.0
    gate: bool = True
    moe: Optional[MoeDef] = None

    def to_json(self):
        d = {"name": self.name, "hidden_dim": self.hidden_dim,
             "activation": _ACT_TO_JSON[self.activation], "bias": self.bias,
             "dropout": float(self.dropout), "gate": self.gate}
        if self.moe is not None:
            d["moe"] = self.moe.to_json()
        return d

    @staticmethod
    def from_json(d) -> "FfnDef":
        moe = d.get("moe")
        return FfnDef(d["name"], d.get("hidden_dim"), _ACT_FROM_JSON[d["activation"]],
                      bool(d["bias"]), float(d["dropout"]), bool(d["gate"]),
                      MoeDef.from_json(moe) if moe is not None else None)


@dataclass
class ReserveExpertsDef:
    capacity: int = 0
    rank: int = 0
    top_k: int = 0

    def to_json(self):
        return {"capacity": self.capacity, "rank": self.rank, "top_k": self.top_k}

    @staticmethod
    def from_json(d):
        return ReserveExpertsDef(int(d["capacity"]), int(d["rank"]), int(d["top_k"]))


@dataclass
class MemoryTierDef:
    name: str
    ffn: FfnDef
    reserve_experts: ReserveExpertsDef
    residual_init: str = "default"      # default | zero

    def to_json(self):
        return {"name": self.name, "ffn": self.ffn.to_json(),
                "reserve_experts": self.reserve_experts.to_json(),
                "residual_init": "ResidualZero" if self.residual_init == "zero" else "Default"}

    @staticmethod
    def from_json(d):
        return MemoryTierDef(d["name"], FfnDef.from_json(d["ffn"]),
                             ReserveExpertsDef.from_json(d["reserve_experts"]),
                             "zero" if d.get("residual_init", "Default") == "ResidualZero" else "default")


@dataclass
class MemoryDef:
    name: str
    tiers: List[MemoryTierDef]

    def to_json(self):
        return {"name": self.name, "tiers": [t.to_json() for t in self.tiers]}

    @staticmethod
    def from_json(d):
        return MemoryDef(d["name"], [MemoryTierDef.from_json(t) for t in d["tiers"]])


_NORM_TO_JSON = {"rmsnorm": "RmsNorm", "layernorm": "LayerNorm", "none": "None"}
_NORM_FROM_JSON = {v: k for k, v in _NORM_TO_JSON.items()}


@dataclass
class NormConfig:
    norm_type: str = "rmsnorm"
    eps: float = 0.0

    def to_json(self):
        return {"norm_type": _NORM_TO_JSON[self.norm_type], "eps": float(self.eps)}

    @staticmethod
    def from_json(d):
        return NormConfig(_NORM_FROM_JSON[d["norm_type"]], float(d["eps"]))

    def effective_eps(self) -> float:
        return self.eps if self.eps > 0.0 else 1e-5


@dataclass
class BlockDef:
    name: str = "default"
    attention: AttentionDef = field(default_factory=AttentionDef)
    ssm: Optional[SsmDef] = None
    ffn: FfnDef = field(default_factory=FfnDef)
    memory: Optional[MemoryDef] = None
    norm: NormConfig = field(default_factory=lambda: NormConfig("rmsnorm", 1e-5))
    norm_position: str = "pre"
    residual: bool = True
    dropout: float = 0.0

    # per-block derived properties (summa-mal/src/lib.rs:324-376)
    def is_ssm(self) -> bool:
        return self.ssm is not None

    def num_heads(self) -> int:
        return self.attention.num_heads if self.attention.num_heads is not None else 12

    def num_kv_heads(self) -> int:
        kv = self.attention.num_kv_heads
        return kv if kv is not None else self.num_heads()

    def head_dim(self, hidden_size: int) -> int:
        hd = self.attention.head_dim
        return hd if hd is not None else hidden_size // self.num_heads()

    def intermediate_size(self, hidden_size: int) -> int:
        return self.ffn.hidden_dim if self.ffn.hidden_dim is not None else hidden_size * 4

    def norm_eps(self) -> float:
        return self.norm.effective_eps()

    def rope_theta(self) -> float:
        pe = self.attention.position_encoding
        return pe.theta if pe.kind == "rope" else 10000.0

    def rope_scaling(self) -> Optional[float]:
        pe = self.attention.position_encoding
        return pe.scaling if pe.kind == "rope" else None

    def to_json(self):
        d = {"name": self.name, "attention": self.attention.to_json(),
             "ssm": self.ssm.to_json() if self.ssm else None,
             "ffn": self.ffn.to_json()}
        if self.memory is not None:
            d["memory"] = self.memory.to_json()
        d.update({"norm": self.norm.to_json(),
                  "norm_position": "Pre" if self.norm_position == "pre" else "Post",
                  "residual": self.residual, "dropout": float(self.dropout)})
        return d

    @staticmethod
    def from_json(d) -> "BlockDef":
        ssm = d.get("ssm")
        mem = d.get("memory")
        return BlockDef(
            name=d["name"], attention=AttentionDef.from_json(d["attention"]),
            ssm=SsmDef.from_json(ssm) if ssm is not None else None,
            ffn=FfnDef.from_json(d["ffn"]),
            memory=MemoryDef.from_json(mem) if mem is not None else None,
            norm=NormConfig.from_json(d["norm"]),
            norm_position="pre" if d["norm_position"] == "Pre" else "post",
            residual=bool(d["residual"]), dropout=float(d["dropout"]))


@dataclass
class EmbeddingsConfig:
    tie_weights: bool = False
    dropout: float = 0.0
    scale: Optional[float] = None

    def to_json(self):
        return {"tie_weights": self.tie_weights, "dropout": float(self.dropout),
                "scale": self.scale}

    @staticmethod
    def from_json(d):
        return EmbeddingsConfig(bool(d["tie_weights"]), float(d["dropout"]), d.get("scale"))


@dataclass
class OutputConfig:
    bias: bool = False
    norm: Optional[NormConfig] = None

    def to_json(self):
        return {"bias": self.bias, "norm": self.norm.to_json() if self.norm else None}

    @staticmethod
    def from_json(d):
        n = d.get("norm")
        return OutputConfig(bool(d["bias"]), NormConfig.from_json(n) if n is not None else None)


def _next_multiple_of(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass
class ModelDef:
    name: str = "default"
    description: Optional[str] = None
    vocab_size: int = 32000
    max_seq_len: int = 2048
    hidden_size: int = 768
    num_layers: int = 12
    block: BlockDef = field(default_factory=BlockDef)
    pattern: Optional[List[BlockDef]] = None
    embeddings: EmbeddingsConfig = field(default_factory=EmbeddingsConfig)
    output: OutputConfig = field(default_factory=OutputConfig)

    def block_for_layer(self, i: int) -> BlockDef:
        if self.pattern:
            return self.pattern[i % len(self.pattern)]
        return self.block

    def dt_rank(self, ssm: SsmDef) -> int:
        return ssm.dt_rank if ssm.dt_rank is not None else -(-self.hidden_size // 16)

    def padded_vocab_size(self) -> int:
        """Rows stored by the embedding / head: logical vocab rounded up to 64."""
        return _next_multiple_of(self.vocab_size, 64)

    def estimated_params(self) -> int:
        """Exact trainable-parameter count (summa-mal/src/lib.rs:582-666)."""
        h = self.hidden_size
        vpad = self.padded_vocab_size()

        def norm_params(n: NormConfig) -> int:
            return {"rmsnorm": h, "layernorm": 2 * h, "none": 0}[n.norm_type]

        def ffn_params(f: FfnDef) -> int:
            inter = f.hidden_dim if f.hidden_dim is not None else 4 * h
            proj = 3 if f.gate else 2
            n_exp = (f.moe.experts + f.moe.shared_experts) if f.moe else 1
            w = n_exp * proj * h * inter
            b = n_exp * ((2 if f.gate else 1) * inter + h) if f.bias else 0
            router = h * f.moe.experts if f.moe else 0
            return w + b + router

        total = 0
        for i in range(self.num_layers):
            blk = self.block_for_layer(i)
            if blk.ssm is not None:
                s = blk.ssm
                di = s.expand * h
                r = self.dt_rank(s)
                mixer = (2 * h * di + di * h + di * s.conv_kernel
                         + di * (r + 2 * s.state_dim) + r * di + di
                         + di * s.state_dim + di + di)
            else:
                q = blk.num_heads() * blk.head_dim(h)
                kv = blk.num_kv_heads() * blk.head_dim(h)
                mixer = h * q + 2 * h * kv + q * h
                if blk.attention.bias:
                    mixer += 2 * q + 2 * kv
                if blk.attention.qk_norm:
                    mixer += 2 * blk.head_dim(h)
            if blk.memory is not None:
                ff = sum(ffn_params(t.ffn)
                         + t.reserve_experts.capacity * (2 * h * t.reserve_experts.rank + h)
                         for t in blk.memory.tiers)
            else:
                ff = ffn_params(blk.ffn)
            total += mixer + ff + 2 * norm_params(blk.norm)
        final_norm = self.output.norm or self.block_for_layer(0).norm
        head_w = 0 if self.embeddings.tie_weights else h * vpad
        head_b = vpad if self.output.bias else 0
        return vpad * h + total + norm_params(final_norm) + head_w + head_b

    def to_json(self) -> dict:
        return {
            "name": self.name, "description": self.description,
            "vocab_size": self.vocab_size, "max_seq_len": self.max_seq_len,
            "hidden_size": self.hidden_size, "num_layers": self.num_layers,
            "block": self.block.to_json(),
            "pattern": [b.to_json() for b in self.pattern] if self.pattern else None,
            "embeddings": self.embeddings.to_json(), "output": self.output.to_json(),
        }

    def to_json_str(self) -> str:
        return json.dumps(self.to_json(), indent=2)

    def save_json(self, path: str) -> None:
        with open(path, "w") as f:
            f.write(self.to_json_str())

    @staticmethod
    def from_json(d) -> "ModelDef":
        if isinstance(d, (str, bytes)):
            d = json.loads(d)
        pat = d.get("pattern")
        return ModelDef(
            name=d["name"], description=d.get("description"),
            vocab_size=int(d["vocab_size"]), max_seq_len=int(d["max_seq_len"]),
            hidden_size=int(d["hidden_size"]), num_layers=int(d["num_layers"]),
            block=BlockDef.from_json(d["block"]),
            pattern=[BlockDef.from_json(b) for b in pat] if pat else None,
            embeddings=EmbeddingsConfig.from_json(d["embeddings"]),
            output=OutputConfig.from_json(d["output"]))


@dataclass
class MalFile:
    attentions: Dict[str, AttentionDef] = field(default_factory=dict)
    ssms: Dict[str, SsmDef] = field(default_factory=dict)
    ffns: Dict[str, FfnDef] = field(default_factory=dict)
    memories: Dict[str, MemoryDef] = field(default_factory=dict)
    blocks: Dict[str, BlockDef] = field(default_factory=dict)
    models: Dict[str, ModelDef] = field(default_factory=dict)


# --------------------------------------------------------------------------
# Lexer
# --------------------------------------------------------------------------

_TOKEN_RE = re.compile(r"""
    (?P<ws>[ \t\r\n]+|\#[^\n]*)
  | (?P<number>-?[0-9]+(?:\.[0-9]+)?(?:[eE][+-]?[0-9]+)?)
  | (?P<ident>[A-Za-z_][A-Za-z0-9_\-]*)
  | (?P<string>"(?:[^"\\]|\\.)*")
  | (?P<punct>[{}\[\]:,])
""", re.VERBOSE | re.DOTALL)


class _Lexer:
    def __init__(self, src: str):
        self.toks = []
        pos = 0
        line = 1
        while pos < len(src):
            m = _TOKEN_RE.match(src, pos)
            if not m:
                raise MalError(f"Parse error: unexpected character {src[pos]!r} at line {line}")
            kind = m.lastgroup
            text = m.group(0)
            if kind != "ws":
                self.toks.append((kind, text, line))
            line += text.count("\n")
            pos = m.end()
        self.toks.append(("eof", "", line))
        self.i = 0

    def peek(self, k=0):
        return self.toks[min(self.i + k, len(self.toks) - 1)]

    def next(self):
        t = self.toks[self.i]
        self.i += 1
        return t

    def err(self, msg):
        kind, text, line = self.peek()
        raise MalError(f"Parse error: {msg} at line {line} (found {text!r})")

    def expect(self, text):
        t = self.next()
        if t[1] != text or t[0] == "string":
            self.i -= 1
            self.err(f"expected {text!r}")
        return t

    def accept(self, text):
        t = self.peek()
        if t[1] == text and t[0] != "string":
            self.i += 1
            return True
        return False

    def ident(self):
        t = self.next()
        if t[0] != "ident":
            self.i -= 1
            self.err("expected identifier")
        return t[1]

    def integer(self) -> int:
        t = self.next()
        if t[0] != "number" or not t[1].isdigit():
            self.i -= 1
            self.err("expected integer")
        return int(t[1])

    def number(self) -> float:
        t = self.next()
        if t[0] != "number":
            self.i -= 1
            self.err("expected number")
        return float(t[1])

    def boolean(self) -> bool:
        t = self.next()
        if t[1] not in ("true", "false") or t[0] != "ident":
            self.i -= 1
            self.err("expected boolean")
        return t[1] == "true"


# --------------------------------------------------------------------------
# Parser
# --------------------------------------------------------------------------

def _props(lx: _Lexer, handler) -> None:
    """Parse `{ prop* }` calling handler(key) for every property keyword."""
    lx.expect("{")
    while not lx.accept("}"):
        kind, text, _ = lx.peek()
        if kind != "ident":
            lx.err("expected property name")
        lx.next()
        if not handler(text):
            lx.i -= 1
            lx.err(f"unknown property {text!r}")


def _parse_position_encoding(lx: _Lexer) -> PositionEncoding:
    which = lx.ident()
    if which == "none":
        return PositionEncoding(kind="none")
    if which == "rope":
        pe = PositionEncoding(kind="rope")

        def h(key):
            if key in ("rope_theta", "theta", "base"):
                lx.expect(":"); pe.theta = lx.number(); return True
            if key == "rope_scaling":
                lx.expect(":"); pe.scaling = lx.number(); return True
            return False
        _props(lx, h)
        return pe
    if which == "alibi":
        pe = PositionEncoding(kind="alibi")

        def h(key):
            if key == "slopes":
                lx.expect(":")
                v = lx.ident()
                if v not in ("learned", "fixed"):
                    lx.i -= 1; lx.err("expected learned|fixed")
                pe.learned_slopes = v == "learned"
                return True
            return False
        _props(lx, h)
        return pe
    if which == "learned":
        pe = PositionEncoding(kind="learned")

        def h(key):
            if key == "max_positions":
                lx.expect(":"); pe.max_positions = lx.integer(); return True
            return False
        _props(lx, h)
        return pe
    lx.i -= 1
    lx.err("expected rope|alibi|learned|none")


def _attention_handler(lx: _Lexer, a: AttentionDef):
    def h(key):
        if key in ("num_heads", "n_heads", "attention_heads"):
            lx.expect(":"); a.num_heads = lx.integer()
        elif key in ("num_kv_heads", "kv_heads"):
            lx.expect(":"); a.num_kv_heads = lx.integer()
        elif key == "head_dim":
            lx.expect(":"); a.head_dim = lx.integer()
        elif key == "dropout":
            lx.expect(":"); a.dropout = lx.number()
        elif key == "bias":
            lx.expect(":"); a.bias = lx.boolean()
        elif key == "position_encoding":
            lx.expect(":"); a.position_encoding = _parse_position_encoding(lx)
        elif key == "window_size":
            lx.expect(":"); a.window_size = lx.integer()
        elif key == "causal":
            lx.expect(":"); a.causal = lx.boolean()
        elif key == "qk_norm":
            lx.expect(":"); a.qk_norm = lx.boolean()
        else:
            return False
        return True
    return h


_ACTIVATIONS = ("swiglu", "gelu", "silu", "relu", "gelu_new", "gelu_tanh")


def _ffn_handler(lx: _Lexer, f: FfnDef):
    def h(key):
        if key in ("hidden_dim", "intermediate_size"):
            lx.expect(":"); f.hidden_dim = lx.integer()
        elif key == "activation":
            lx.expect(":")
            v = lx.ident()
            if v not in _ACTIVATIONS:
                lx.i -= 1; lx.err("unknown activation")
            f.activation = v
        elif key == "bias":
            lx.expect(":"); f.bias = lx.boolean()
        elif key == "dropout":
            lx.expect(":"); f.dropout = lx.number()
        elif key == "gate":
            lx.expect(":"); f.gate = lx.boolean()
        elif key == "moe":
            moe = MoeDef()

            def mh(k):
                if k == "experts":
                    lx.expect(":"); moe.experts = lx.integer()
                elif k == "top_k":
                    lx.expect(":"); moe.top_k = lx.integer()
                elif k == "shared_experts":
                    lx.expect(":"); moe.shared_experts = lx.integer()
                elif k == "load_balance_loss_weight":
                    lx.expect(":"); moe.load_balance_loss_weight = lx.number()
                elif k == "router_z_loss_weight":
                    lx.expect(":"); moe.router_z_loss_weight = lx.number()
                else:
                    return False
                return True
            _props(lx, mh)
            f.moe = moe
        else:
            return False
        return True
    return h


def _ssm_handler(lx: _Lexer, s: SsmDef):
    def h(key):
        if key in ("state_dim", "d_state"):
            lx.expect(":"); s.state_dim = lx.integer()
        elif key in ("conv_kernel", "d_conv"):
            lx.expect(":"); s.conv_kernel = lx.integer()
        elif key == "expand":
            lx.expect(":"); s.expand = lx.integer()
        elif key == "dt_rank":
            lx.expect(":"); s.dt_rank = lx.integer()
        else:
            return False
        return True
    return h


def _parse_norm_config(lx: _Lexer) -> NormConfig:
    which = lx.ident()
    if which == "none":
        return NormConfig("none", 0.0)
    if which not in ("rmsnorm", "layernorm"):
        lx.i -= 1
        lx.err("expected rmsnorm|layernorm|none")
    n = NormConfig(which, 0.0)

    def h(key):
        if key in ("norm_eps", "eps"):
            lx.expect(":"); n.eps = lx.number(); return True
        return False
    _props(lx, h)
    return n


def _parse_memory_tiers(lx: _Lexer, file: MalFile) -> List[MemoryTierDef]:
    lx.expect("{")
    tiers = []
    while not lx.accept("}"):
        lx.expect("tier")
        name = lx.ident()
        state = {"ffn": None, "reserve": None, "init": "default"}

        def h(key):
            if key == "ffn":
                lx.expect(":")
                if lx.peek()[1] == "{":
                    f = FfnDef()
                    _props(lx, _ffn_handler(lx, f))
                    state["ffn"] = f
                else:
                    ref = lx.ident()
                    if ref not in file.ffns:
                        raise MalError(f"undefined ffn '{ref}'")
                    state["ffn"] = _clone(file.ffns[ref])
            elif key == "reserve_experts":
                r = ReserveExpertsDef()

                def rh(k):
                    if k == "capacity":
                        lx.expect(":"); r.capacity = lx.integer()
                    elif k == "rank":
                        lx.expect(":"); r.rank = lx.integer()
                    elif k == "top_k":
                        lx.expect(":"); r.top_k = lx.integer()
                    else:
                        return False
                    return True
                _props(lx, rh)
                state["reserve"] = r
            elif key == "residual_init":
                lx.expect(":")
                v = lx.ident()
                if v not in ("default", "zero"):
                    lx.i -= 1; lx.err("expected default|zero")
                state["init"] = v
            else:
                return False
            return True
        _props(lx, h)
        if state["ffn"] is None:
            raise MalError("memory tier requires an ffn")
        if state["reserve"] is None:
            raise MalError("memory tier requires reserve_experts")
        tiers.append(MemoryTierDef(name, state["ffn"], state["reserve"], state["init"]))
    if not tiers:
        lx.err("memory requires at least one tier")
    return tiers


def _clone(x):
    import copy
    return copy.deepcopy(x)


def _block_handler(lx: _Lexer, b: BlockDef, file: MalFile):
    def ref_or_inline(table, kind, make, handler_factory):
        lx.expect(":")
        if lx.peek()[1] == "{":
            obj = make()
            _props(lx, handler_factory(lx, obj))
            return obj
        name = lx.ident()
        if name not in table:
            raise MalError(f"undefined {kind} '{name}'")
        return _clone(table[name])

    def h(key):
        if key == "attention":
            b.attention = ref_or_inline(file.attentions, "attention", AttentionDef, _attention_handler)
        elif key == "ssm":
            b.ssm = ref_or_inline(file.ssms, "ssm", SsmDef, _ssm_handler)
        elif key == "ffn":
            b.ffn = ref_or_inline(file.ffns, "ffn", FfnDef, _ffn_handler)
        elif key == "memory":
            lx.expect(":")
            if lx.peek()[1] == "{":
                b.memory = MemoryDef("default", _parse_memory_tiers(lx, file))
            else:
                name = lx.ident()
                if name not in file.memories:
                    raise MalError(f"undefined memory '{name}'")
                b.memory = _clone(file.memories[name])
        elif key == "norm":
            lx.expect(":"); b.norm = _parse_norm_config(lx)
        elif key == "norm_position":
            lx.expect(":")
            v = lx.ident()
            if v not in ("pre", "post"):
                lx.i -= 1; lx.err("expected pre|post")
            b.norm_position = v
        elif key == "residual":
            lx.expect(":"); b.residual = lx.boolean()
        elif key == "dropout":
            lx.expect(":"); b.dropout = lx.number()
        else:
            return False
        return True
    return h


def _model_handler(lx: _Lexer, m: ModelDef, file: MalFile):
    def h(key):
        if key == "vocab_size":
            lx.expect(":"); m.vocab_size = lx.integer()
        elif key in ("max_seq_len", "context_length", "seq_len"):
            lx.expect(":"); m.max_seq_len = lx.integer()
        elif key in ("hidden_size", "d_model", "embed_dim"):
            lx.expect(":"); m.hidden_size = lx.integer()
        elif key in ("num_layers", "n_layers", "depth"):
            lx.expect(":"); m.num_layers = lx.integer()
        elif key == "block":
            lx.expect(":")
            if lx.peek()[1] == "{":
                blk = BlockDef()
                _props(lx, _block_handler(lx, blk, file))
                m.block = blk
            else:
                name = lx.ident()
                if name not in file.blocks:
                    raise MalError(f"undefined block '{name}'")
                m.block = _clone(file.blocks[name])
        elif key == "pattern":
            lx.expect(":"); lx.expect("[")
            blocks = []
            while True:
                name = lx.ident()
                if name not in file.blocks:
                    raise MalError(f"pattern references undefined block '{name}'")
                blocks.append(_clone(file.blocks[name]))
                if lx.accept(","):
                    if lx.accept("]"):
                        break
                    continue
                lx.expect("]")
                break
            m.pattern = blocks
        elif key == "embeddings":
            def eh(k):
                if k == "tie_weights":
                    lx.expect(":"); m.embeddings.tie_weights = lx.boolean()
                elif k == "dropout":
                    lx.expect(":"); m.embeddings.dropout = lx.number()
                elif k == "scale":
                    lx.expect(":"); m.embeddings.scale = lx.number()
                else:
                    return False
                return True
            _props(lx, eh)
        elif key == "output":
            def oh(k):
                if k == "bias":
                    lx.expect(":"); m.output.bias = lx.boolean()
                elif k == "norm":
                    lx.expect(":"); m.output.norm = _parse_norm_config(lx)
                else:
                    return False
                return True
            _props(lx, oh)
        elif key == "description":
            lx.expect(":")
            t = lx.next()
            if t[0] != "string":
                lx.i -= 1; lx.err("expected quoted string")
            m.description = t[1][1:-1]
        else:
            return False
        return True
    return h


def _insert_unique(table: dict, kind: str, name: str, value) -> None:
    if name in table:
        raise MalError(f"duplicate {kind} '{name}'")
    table[name] = value


def parse_mal_full(source: str) -> MalFile:
    """Parse a MAL source with any number of definitions.

    References resolve against definitions that appear EARLIER in the file,
    like the reference's single forward pass (`summa-mal/src/lib.rs:889-960`).
    """
    lx = _Lexer(source)
    file = MalFile()
    if lx.peek()[0] == "eof":
        lx.err("expected at least one definition")
    while lx.peek()[0] != "eof":
        kw = lx.ident()
        if kw == "attention":
            a = AttentionDef(name=lx.ident())
            _props(lx, _attention_handler(lx, a))
            _insert_unique(file.attentions, "attention", a.name, a)
        elif kw == "ffn":
            f = FfnDef(name=lx.ident())
            _props(lx, _ffn_handler(lx, f))
            _insert_unique(file.ffns, "ffn", f.name, f)
        elif kw == "ssm":
            s = SsmDef(name=lx.ident())
            _props(lx, _ssm_handler(lx, s))
            _insert_unique(file.ssms, "ssm", s.name, s)
        elif kw == "memory":
            name = lx.ident()
            mem = MemoryDef(name, _parse_memory_tiers(lx, file))
            _insert_unique(file.memories, "memory", name, mem)
        elif kw == "block":
            b = BlockDef(name=lx.ident())
            _props(lx, _block_handler(lx, b, file))
            _insert_unique(file.blocks, "block", b.name, b)
        elif kw == "model":
            m = ModelDef(name=lx.ident())
            _props(lx, _model_handler(lx, m, file))
            _insert_unique(file.models, "model", m.name, m)
        else:
            lx.i -= 1
            lx.err("expected attention|ffn|ssm|memory|block|model")
    return file


def parse_mal(source: str) -> ModelDef:
    """Parse a MAL source that defines exactly one model."""
    file = parse_mal_full(source)
    if not file.models:
        raise MalError("no model definition found")
    if len(file.models) > 1:
        raise MalError("multiple model definitions found (%s); use parse_mal_full to select one"
                       % ", ".join(sorted(file.models)))
    return next(iter(file.models.values()))


def parse_mal_file(path: str) -> ModelDef:
    with open(path, "r", encoding="utf-8") as f:
        return parse_mal(f.read())


_WELL_KNOWN_DIR = os.path.join(os.path.dirname(__file__), "well_known")


def list_wellknown_models() -> List[str]:
    return sorted(os.path.splitext(n)[0] for n in os.listdir(_WELL_KNOWN_DIR) if n.endswith(".mal"))


def get_builtin_model(name: str) -> ModelDef:
    """Preset lookup; accepts the file stem with `-` or `_` separators."""
    stem = name.replace("-", "_")
    path = os.path.join(_WELL_KNOWN_DIR, stem + ".mal")
    if not os.path.exists(path):
        raise MalError(f"unknown built-in model '{name}' (available: {', '.join(list_wellknown_models())})")
    return parse_mal_file(path)


def load_model_def(path_or_name: str) -> ModelDef:
    """`.mal` file, `ModelDef` JSON file, or preset name."""
    if os.path.exists(path_or_name):
        if path_or_name.endswith(".json"):
            with open(path_or_name) as f:
                return ModelDef.from_json(json.load(f))
        return parse_mal_file(path_or_name)
    return get_builtin_model(path_or_name)
