"""The reference's checkpoint format (meta.json + params.npz, benchmarking.py:100-145) and the
scoring path over it (model.eval_logprobs, benchmarking.Scorer)."""

import json
import os

import numpy as np
import pytest
import torch

from algebraic_transformer_b200 import checkpoint as C
from algebraic_transformer_b200 import prefill as P
from oracle import algebraic_ref as R
from oracle import model_ref as M

CFG = P.PrefillConfig(vocab_size=1000, d_model=128, n_layers=2, n_heads=2, d_ff=256, alu_beta=0.5, attn_n=16,
                      attn_c=8.0, head_n=8, head_c=2.0)


def _params(seed=0):
    p = P.init_params(CFG, seed=seed)
    g = torch.Generator().manual_seed(seed + 1)
    for k in ("q_gain", "k_gain"):
        p[k] = 0.75 + 0.5 * torch.rand(p[k].shape, generator=g)
    p["sink"] = torch.randn(p["sink"].shape, generator=g) * 0.3
    return p


def test_checkpoint_round_trip_and_validation(tmp_path):
    run = str(tmp_path / "run")
    params = _params()
    C.save_checkpoint(run, CFG, params, seq_len=256)
    with np.load(os.path.join(run, "params.npz")) as flat:       # the reference's key strings
        assert "['embed']" in flat.files and "['layers']['w_q']" in flat.files and len(flat.files) == 15
    cfg, seq_len, got = C.load_checkpoint(run)
    assert cfg == CFG and seq_len == 256
    assert set(got) == set(params) and all(torch.equal(got[k], params[k].float()) for k in params)

    def rewrite(mutate):
        with np.load(os.path.join(run, "params.npz")) as flat:
            d = {k: flat[k] for k in flat.files}
        mutate(d)
        np.savez(os.path.join(run, "params.npz"), **d)

    rewrite(lambda d: d.update({"['layers']['w_x']": np.zeros(3, np.float32)}))
    with pytest.raises(ValueError, match="unexpected"):
        C.load_checkpoint(run)
    rewrite(lambda d: (d.pop("['layers']['w_x']"), d.update({"['embed']": d["['embed']"][:, :64]})))
    with pytest.raises(ValueError, match="invalid"):
        C.load_checkpoint(run)
    C.save_checkpoint(run, CFG, params, seq_len=256)
    rewrite(lambda d: d["['layers']['sink']"].__setitem__((0, 0), np.nan))
    with pytest.raises(ValueError, match="invalid"):
        C.load_checkpoint(run)
    C.save_checkpoint(run, CFG, params, seq_len=256)
    rewrite(lambda d: d.pop("['final_gain']"))
    with pytest.raises(ValueError, match="missing"):
        C.load_checkpoint(run)
    # a softmax-attention checkpoint is not something these kernels serve
    C.save_checkpoint(run, CFG, params, seq_len=256)
    meta = json.load(open(os.path.join(run, "meta.json")))
    meta["config"]["attn"] = "softmax"
    json.dump(meta, open(os.path.join(run, "meta.json"), "w"))
    with pytest.raises(ValueError, match="algebraic preset"):
        C.load_checkpoint(run)


@pytest.mark.gpu
def test_scoring_matches_oracle(tmp_path):
    run = str(tmp_path / "run")
    C.save_checkpoint(run, CFG, _params(3), seq_len=256)
    cfg, seq_len, params = C.load_checkpoint(run)
    scorer = C.Scorer(cfg, params, "cuda:0", seq_len=seq_len, batch=4)
    g = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, cfg.vocab_size, (2, 256), generator=g)
    targets = torch.roll(tokens, -1, dims=1)
    hid = M.forward_hidden(params, tokens, cfg)
    _, pt = M.head_loss(params, hid, targets, cfg)
    want = torch.log(pt).view(2, 256)
    got = scorer.eval_logprobs(tokens, targets).cpu()
    assert float((got - want).abs().max()) < 0.08 and float((got - want).norm() / want.norm()) < 1e-2
    # continuation scoring with the reference's semantics (benchmarking.py:196-240): the model sees
    # context + cont[:-1]; the score is the MEAN log p over the continuation plus the greedy-match flag
    pairs = [(tokens[0, :40].tolist(), tokens[0, 40:47].tolist()), (tokens[1, :100].tolist(), tokens[1, 100:103].tolist()),
             (tokens[0, :5].tolist(), tokens[0, 5:6].tolist()),
             (tokens[1, :250].tolist(), tokens[1, 250:256].tolist() + [7])]    # context + continuation == T + 1 tokens
    scores, hits = scorer.score_token_pairs(pairs)
    assert len(scores) == len(hits) == len(pairs)
    for (ctx, cont), s, hit in zip(pairs, scores, hits):
        seq = torch.tensor([ctx + cont[:-1]])
        n = seq.shape[1]
        bucket = min(256, max(128, 1 << (n - 1).bit_length()))
        x = torch.zeros((1, bucket), dtype=torch.long)
        x[0, :n] = seq
        h = M.forward_hidden(params, x, cfg)[0, len(ctx) - 1:n]
        _, pt_c = R.head_loss_dense(h, params["embed"], torch.tensor(cont), cfg.head_n, cfg.head_c)
        want_s = float(torch.log(pt_c).mean())
        assert abs(s - want_s) < 0.05 * max(1.0, abs(want_s))
        z = R.head_logits(h, params["embed"])
        top2 = z.topk(2, dim=-1).values
        if float((top2[:, 0] - top2[:, 1]).min()) > 0.05:       # unambiguous arg-max rows only
            assert hit == bool(torch.equal(z.argmax(-1), torch.tensor(cont)))
    # a context that does not fit is an error unless truncation is allowed
    long_pair = [(tokens[0].tolist() + tokens[1, :10].tolist(), tokens[1, 10:13].tolist())]
    with pytest.raises(ValueError, match="truncate"):
        scorer.score_token_pairs(long_pair)
    s_trunc, _ = scorer.score_token_pairs(long_pair, allow_truncation=True)
    assert scorer.truncated_pairs == 1 and np.isfinite(s_trunc[0])
