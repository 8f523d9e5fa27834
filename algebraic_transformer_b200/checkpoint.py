"""The reference's on-disk checkpoint (`meta.json` + `params.npz`) and its scoring path, so that a
run directory written by the reference's trainer can be scored on a B200.

Format (src/algebraic/train.py:422-428, src/algebraic/benchmarking.py:100-145): `params.npz` holds the
parameter tree flattened with `jax.tree_util.keystr`, i.e. keys like `['embed']` and
`['layers']['w_q']`; `meta.json` carries the `LMConfig` fields under `"config"`.  Only the
`algebraic` preset is served (RMS norm, ALU-GLU, Cayley positions, QK-norm, asinh attention with a
learned sink, Alg-CE head): those are the kernels this package has.

Scoring (src/algebraic/model.py:238-247, benchmarking.py:170-190): per-token `log p(target)` under
the head's normalised distribution.  For the Alg-CE head that is `log(w_t / sum_j w_j)`, which the
fused head kernel already returns as its NLL telemetry, so no `[tokens x vocab]` logits are formed
here either; `score_token_pairs` projects the continuation positions only, as the reference does.
"""

import json
import os
import re
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

from .prefill import Prefill, PrefillConfig

_PRESET = {"norm": "rms", "ffn": "alu_glu", "pos": "cayley_geo", "attn": "asinh", "sink": "learned", "head": "alg_ce",
           "qk_norm": True}
_LAYER_KEYS = ("w_q", "w_k", "w_v", "w_o", "w_g", "w_u", "w_d", "ln1", "ln2", "q_gain", "k_gain", "sink")
_TOP_KEYS = ("embed", "embed_gain", "final_gain")


def _expected_shapes(cfg: PrefillConfig) -> Dict[Tuple[str, ...], Tuple[int, ...]]:
    L, d, f, H, D = cfg.n_layers, cfg.d_model, cfg.d_ff, cfg.n_heads, cfg.head_dim
    exp = {("embed",): (cfg.vocab_size, d), ("embed_gain",): (d,), ("final_gain",): (d,)}
    for name in ("w_q", "w_k", "w_v", "w_o"):
        exp[("layers", name)] = (L, d, d)
    for name in ("w_g", "w_u"):
        exp[("layers", name)] = (L, d, f)
    exp[("layers", "w_d")] = (L, f, d)
    exp.update({("layers", "ln1"): (L, d), ("layers", "ln2"): (L, d), ("layers", "q_gain"): (L, D),
                ("layers", "k_gain"): (L, D), ("layers", "sink"): (L, H)})
    return exp


def config_from_meta(meta: dict) -> Tuple[PrefillConfig, int]:
    """`(PrefillConfig, seq_len)` from the `"config"` block of a run's meta.json; raises ValueError
    for anything but the algebraic preset."""
    c = meta["config"]
    for key, want in _PRESET.items():
        if c.get(key) != want:
            raise ValueError(f"checkpoint is not the algebraic preset: {key}={c.get(key)!r}, need {want!r}")
    if float(c.get("rope_fraction", 1.0)) != 1.0:
        raise ValueError("partial Cayley rotation (rope_fraction != 1) is not built")
    if c["d_model"] % c["n_heads"]:
        raise ValueError("d_model must be divisible by n_heads")
    cfg = PrefillConfig(vocab_size=int(c["vocab_size"]), d_model=int(c["d_model"]), n_layers=int(c["n_layers"]),
                        n_heads=int(c["n_heads"]), d_ff=int(c["d_ff"]), eps=float(c.get("eps", 1e-5)),
                        alu_beta=float(c.get("alu_beta", 1.0)), rope_base=float(c.get("rope_base", 10000.0)),
                        attn_n=int(c.get("attn_n", 8)), attn_c=float(c.get("attn_c", 1.0)),
                        head_n=int(c.get("head_n", 16)), head_c=float(c.get("head_c", 16.0)),
                        init_std=float(c.get("init_std", 0.02)))
    return cfg, int(c.get("seq_len", 1024))


def _parse_key(key: str) -> Tuple[str, ...]:
    """`['layers']['w_q']` -> ("layers", "w_q") (the reference flattens its tree with keystr)."""
    return tuple(re.findall(r"\['([^']+)'\]", key))


def load_checkpoint(run_dir: str):
    """`(cfg, seq_len, params)` of a run directory.  The archive is checked as a whole before any
    tensor is kept, against the same rules the reference applies (benchmarking.py:118-145):
    every stored name must be one of the model's parameters and occur once, every parameter must
    be stored, and every array must have the model's shape and hold finite values only; each
    failure raises ValueError.  `params` uses this package's flat layout (`prefill.init_params`)."""
    with open(os.path.join(run_dir, "meta.json")) as f:
        cfg, seq_len = config_from_meta(json.load(f))
    shapes = _expected_shapes(cfg)
    with np.load(os.path.join(run_dir, "params.npz"), allow_pickle=False) as archive:
        names = list(archive.files)
        paths = [_parse_key(name) for name in names]
        strangers = [name for name, path in zip(names, paths) if path not in shapes]
        repeated = [name for name, path in zip(names, paths) if paths.count(path) > 1]
        if strangers or repeated:
            raise ValueError(f"unexpected checkpoint parameter: {(strangers + repeated)[0]}")
        absent = sorted(set(shapes) - set(paths))
        if absent:
            raise ValueError(f"missing checkpoint parameters: {absent}")
        arrays = {path: archive[name] for name, path in zip(names, paths)}
    bad = [path for path, value in arrays.items() if value.shape != shapes[path] or not np.isfinite(value).all()]
    if bad:
        raise ValueError("invalid checkpoint parameter: " + "".join(f"['{part}']" for part in bad[0]))
    params = {path[-1]: torch.from_numpy(np.ascontiguousarray(value, dtype=np.float32)) for path, value in arrays.items()}
    return cfg, seq_len, params


def save_checkpoint(run_dir: str, cfg: PrefillConfig, params: Dict[str, torch.Tensor], seq_len: int = 1024) -> None:
    """Write `params` in the reference's format (the inverse of `load_checkpoint`)."""
    os.makedirs(run_dir, exist_ok=True)
    meta = {"config": dict(_PRESET, vocab_size=cfg.vocab_size, d_model=cfg.d_model, n_layers=cfg.n_layers,
                           n_heads=cfg.n_heads, d_ff=cfg.d_ff, seq_len=int(seq_len), eps=cfg.eps, alu_beta=cfg.alu_beta,
                           rope_base=cfg.rope_base, rope_fraction=1.0, attn_n=cfg.attn_n, attn_c=cfg.attn_c,
                           head_n=cfg.head_n, head_c=cfg.head_c, init_std=cfg.init_std)}
    with open(os.path.join(run_dir, "meta.json"), "w") as f:
        json.dump(meta, f, indent=2)
    flat = {f"['{k}']": params[k].detach().cpu().float().numpy() for k in _TOP_KEYS}
    flat.update({f"['layers']['{k}']": params[k].detach().cpu().float().numpy() for k in _LAYER_KEYS})
    tmp = os.path.join(run_dir, "params.npz.tmp")
    with open(tmp, "wb") as stream:
        np.savez(stream, **flat)
    os.replace(tmp, os.path.join(run_dir, "params.npz"))


class Scorer:
    """Per-token log-probabilities and continuation scores of a loaded model on one GPU
    (benchmarking.Scorer without the tokenizer: it takes token ids)."""

    def __init__(self, cfg: PrefillConfig, params, device, seq_len: int = 1024, batch: int = 8):
        if batch < 1:
            raise ValueError("batch must be positive")
        self.cfg, self.params, self.device, self.T, self.batch = cfg, params, torch.device(device), int(seq_len), batch
        self._models = {}
        self.truncated_pairs = 0

    def _bucket(self, n: int) -> int:
        if n > self.T:
            raise ValueError(f"{n} tokens exceed trained context {self.T}")
        return min(self.T, max(128, 1 << (n - 1).bit_length()))

    def _model(self, bucket: int) -> Prefill:
        # one model serves every bucket: the position tables are built for the trained context
        # and a shorter sequence reads their first rows
        if not self._models:
            self._models[0] = Prefill(self.cfg, self.params, self.device, seq_len=self.T)
        return self._models[0]

    def eval_logprobs(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """`log p(target)` at every position: (B, T) float32 (model.eval_logprobs)."""
        B, T = tokens.shape
        _, _, nll = self._model(T).loss(tokens.to(self.device), targets.to(self.device), want_nll=True)
        return (-nll).view(B, T)

    def score_token_pairs(self, pairs: Sequence[Tuple[List[int], List[int]]], *, allow_truncation: bool = False):
        """`(mean log p, greedy hit)` per (context ids, continuation ids) pair, as the reference's
        `Scorer.score_token_pairs` returns them (benchmarking.py:196-240): the mean of
        `log p(cont[j] | context, cont[:j])` over the continuation, and whether the arg-max token
        equals the target at every continuation position (for a causal model that is the greedy
        generation reproducing the continuation).  The model is fed `context + cont[:-1]`; a
        context too long for the trained length is an error unless `allow_truncation`, which
        keeps its tail and counts the pair in `truncated_pairs`.  Only the continuation positions
        go through the head: `log p` comes from the fused Alg-CE kernel (no logits in HBM for it);
        the arg-max needs the logits of those few rows, one small GEMM.  `log p` is floored at
        log(1e-30) by the kernel's telemetry; non-finite values raise ValueError."""
        from . import ops
        encoded = []
        for context, continuation in pairs:
            ctx, cont = list(context), list(continuation)
            if not ctx or not cont or len(cont) > self.T:
                raise ValueError("need nonempty context/target and target length <= context")
            room = self.T + 1 - len(cont)
            if len(ctx) > room:
                if not allow_truncation:
                    raise ValueError("recall scoring would truncate its evidence")
                ctx = ctx[-room:]
                self.truncated_pairs += 1
            encoded.append((ctx + cont[:-1], len(ctx) - 1, cont))
        lps: List[float] = [0.0] * len(encoded)
        hits: List[bool] = [False] * len(encoded)
        order = sorted(range(len(encoded)), key=lambda i: len(encoded[i][0]))
        for lo in range(0, len(order), self.batch):
            idx = order[lo:lo + self.batch]
            bucket = self._bucket(max(len(encoded[i][0]) for i in idx))
            x = torch.zeros((len(idx), bucket), dtype=torch.long)
            rows, cols, tgt = [], [], []
            for r, i in enumerate(idx):
                seq, start, cont = encoded[i]
                x[r, :len(seq)] = torch.tensor(seq)
                for j, t in enumerate(cont):                    # position start + j predicts cont[j]
                    rows.append(r); cols.append(start + j); tgt.append(t)
            model = self._model(bucket)
            hid = model.hidden(x.to(self.device))
            sel = hid[torch.tensor(rows, device=self.device), torch.tensor(cols, device=self.device)].contiguous()
            n_sel = sel.shape[0]
            pad = (-n_sel) % 8                                   # keep the row count friendly to 16-byte rows
            if pad:
                sel = torch.cat([sel, sel[:1].expand(pad, -1)]).contiguous()
            tg = torch.tensor(tgt + [0] * pad, dtype=torch.int32, device=self.device)
            _, _, nll = ops.fused_head(sel, model.p["embed"], tg, kind="alg_ce", n=self.cfg.head_n, c=self.cfg.head_c,
                                       block_n=sel.shape[0], want_nll=True)
            lp = (-nll[:n_sel]).double().cpu()
            if not bool(torch.isfinite(lp).all()):
                raise ValueError("non-finite evaluation log-probabilities")
            # the head's weight is monotone in the logit, so the arg-max of the logits is the arg-max of p
            top = torch.matmul(sel[:n_sel], model.p["embed"].t()).float().argmax(-1).cpu()
            want = torch.tensor(tgt)
            at = 0
            for r, i in enumerate(idx):
                m = len(encoded[i][2])
                lps[i] = float(lp[at:at + m].mean())
                hits[i] = bool(torch.equal(top[at:at + m], want[at:at + m]))
                at += m
        return lps, hits
