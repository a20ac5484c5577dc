"""A plain, slow Llama: whole sequences, no cache, one function per part.

This file rests on the reference's formulas only: the reference is a Rust
crate and neither `cargo` nor `rustc` exists where these tests run, so its
model code cannot be compiled or imported here.  Each function below restates
one formula and cites where the reference computes it (paths are relative to
the reference project).  Numbers the reference's own unit tests pin down
(RoPE tables, silu(1), the seeded sampling stream) are asserted in
test_plain.py.

Nothing here imports the library under test: a fault in the product cannot
hide by being shared with its oracle.  Everything runs on the CPU with torch
tensors in the dtype the caller picks (float32 by default, float64 to measure
float32's own rounding).
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


# --------------------------------------------------------------------------- rope tables
def plain_inv_freq(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """Inverse frequency per rotated pair, float32[head_dim/2].

    theta^(-2j/rot) in 64-bit from a 32-bit theta, rounded to 32-bit
    (src/config.rs:246-249); then linear (src/config.rs:252-258) or llama3
    (src/config.rs:260-285) rescaling of the rounded entries.
    """
    base = float(np.float32(theta))
    half = head_dim // 2
    inv = [float(np.float32(base ** (-2.0 * j / head_dim))) for j in range(half)]
    kind = None if scaling is None else scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default", "none"):
        pass
    elif kind == "linear":
        s = 1.0 / float(np.float32(scaling["factor"]))
        inv = [float(np.float32(f * s)) for f in inv]
    elif kind == "llama3":
        factor = float(np.float32(scaling["factor"]))
        lo = float(np.float32(scaling.get("low_freq_factor", 1.0)))
        hi = float(np.float32(scaling.get("high_freq_factor", 4.0)))
        orig = float(scaling["original_max_position_embeddings"])
        low_wavelen, high_wavelen = orig / lo, orig / hi
        out = []
        for f in inv:
            wavelen = 2.0 * math.pi / f
            if wavelen < high_wavelen:
                out.append(f)
            elif wavelen > low_wavelen:
                out.append(float(np.float32(f / factor)))
            else:
                smooth = (orig / wavelen - lo) / (hi - lo)
                out.append(float(np.float32((1.0 - smooth) * f / factor + smooth * f)))
        inv = out
    else:
        raise ValueError(f"unknown rope scaling {kind!r}")
    return torch.tensor(inv, dtype=torch.float32)


# --------------------------------------------------------------------------- parts
def plain_embedding(table: torch.Tensor, tokens: Sequence[int], dtype) -> torch.Tensor:
    """x = E[token, :], a row copy without scale (src/model.rs:1237-1242)."""
    return table[torch.tensor(list(tokens), dtype=torch.long)].to(dtype)


def plain_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """ss = sum(x^2)/n + eps; y = x * (1/sqrt(ss)) * w (src/backend/cpu.rs:96-105)."""
    n = x.shape[-1]
    ss = (x * x).sum(dim=-1, keepdim=True) / n + eps
    inv = 1.0 / torch.sqrt(ss)
    return x * inv * weight.to(x.dtype)


def plain_rope(v: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, interleaved: bool) -> torch.Tensor:
    """Rotate the pairs of every head of v[T, heads, head_dim].

    angle = (float32)pos * inv_freq[j], one 32-bit multiply
    (src/backend/cpu.rs:337-338, :346); (x0, x1) <- (x0 c - x1 s, x0 s + x1 c)
    (src/backend/cpu.rs:350-352).  The reference pairs neighbours (2j, 2j+1)
    because its checkpoints ship q/k rows permuted for that; a checkpoint with
    Hugging Face tensor names pairs (j, j + head_dim/2), which the reference
    maps onto the first by permuting rows at load (src/model.rs:1953-1991).
    `interleaved` picks the pairing; the rotation is the same.
    """
    T, H, hd = v.shape
    ang32 = positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, :]
    c = torch.cos(ang32.to(torch.float64)).to(v.dtype)[:, None, :]
    s = torch.sin(ang32.to(torch.float64)).to(v.dtype)[:, None, :]
    out = torch.empty_like(v)
    if interleaved:
        x0, x1 = v[..., 0::2], v[..., 1::2]
        out[..., 0::2] = x0 * c - x1 * s
        out[..., 1::2] = x0 * s + x1 * c
    else:
        half = hd // 2
        x0, x1 = v[..., :half], v[..., half:]
        out[..., :half] = x0 * c - x1 * s
        out[..., half:] = x0 * s + x1 * c
    return out


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0) -> torch.Tensor:
    """Causal grouped-query attention of one whole sequence.

    q[T, H, hd], k and v[T, K, hd].  Query head h reads kv head h // (H/K)
    (src/backend/cpu.rs:385, :395); score = (q.k) / sqrt(hd)
    (src/backend/cpu.rs:386, :413); key t is seen by query r iff t <= r and,
    with a window w > 0, r - t < w (src/backend/cpu.rs:404-409); softmax over
    the seen keys and the weighted sum of their values
    (src/backend/cpu.rs:410-431, written there as an online softmax, which is
    the same function).
    """
    T, H, hd = q.shape
    K = k.shape[1]
    group = H // K
    scale = 1.0 / math.sqrt(hd)
    out = torch.empty_like(q)
    r = torch.arange(T)[:, None]
    t = torch.arange(T)[None, :]
    seen = t <= r
    if window:
        seen &= (r - t) < window
    for h in range(H):
        g = h // group
        scores = (q[:, h, :] @ k[:, g, :].T) * scale
        scores = scores.masked_fill(~seen, float("-inf"))
        p = torch.softmax(scores, dim=-1)
        out[:, h, :] = p @ v[:, g, :]
    return out


def plain_silu(z: torch.Tensor) -> torch.Tensor:
    """silu(z) = z * (1 / (1 + exp(-z))) (src/math.rs:25-27)."""
    return z * (1.0 / (1.0 + torch.exp(-z)))


def plain_swiglu_mlp(xn: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """f = W2 (silu(W1 x) * (W3 x)) (src/model.rs:1336-1345, src/backend/cpu.rs:435-440)."""
    g = xn @ w_gate.to(xn.dtype).T
    u = xn @ w_up.to(xn.dtype).T
    return (plain_silu(g) * u) @ w_down.to(xn.dtype).T


def plain_attention_block(xn, positions, w, prefix, cfg, inv_freq, dtype, window=0):
    """q, k, v = Wq xn, Wk xn, Wv xn; RoPE on q and k; attention; Wo
    (src/model.rs:1253-1301)."""
    H, K, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    T = xn.shape[0]
    q = (xn @ w[prefix + "q_proj.weight"].to(dtype).T).view(T, H, hd)
    k = (xn @ w[prefix + "k_proj.weight"].to(dtype).T).view(T, K, hd)
    v = (xn @ w[prefix + "v_proj.weight"].to(dtype).T).view(T, K, hd)
    q = plain_rope(q, positions, inv_freq, interleaved=False)
    k = plain_rope(k, positions, inv_freq, interleaved=False)
    a = plain_attention(q, k, v, window=window).reshape(T, H * hd)
    return a @ w[prefix + "o_proj.weight"].to(dtype).T


def complete_config(cfg: dict) -> dict:
    """config.json with the derived defaults filled in (src/config.rs:167-173,
    src/model.rs:196-198)."""
    c = dict(cfg)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    if c.get("head_dim") is None:
        c["head_dim"] = c["hidden_size"] // c["num_attention_heads"]
    c.setdefault("rope_theta", 10000.0)
    c.setdefault("rms_norm_eps", 1e-5)
    c.setdefault("tie_word_embeddings", False)
    return c


def plain_hidden(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], dtype=torch.float32) -> torch.Tensor:
    """The residual stream after the last layer, [T, hidden], before the final norm.

    x -> [norm -> attention -> +x] -> [norm -> feed-forward -> +x] per layer
    (src/model.rs:1244-1357).
    """
    cfg = complete_config(cfg)
    inv_freq = plain_inv_freq(cfg["head_dim"], cfg["rope_theta"], cfg.get("rope_scaling"))
    eps = cfg["rms_norm_eps"]
    x = plain_embedding(w["model.embed_tokens.weight"], tokens, dtype)
    positions = torch.arange(len(tokens))
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        xn = plain_rmsnorm(x, w[p + "input_layernorm.weight"], eps)
        x = x + plain_attention_block(xn, positions, w, p + "self_attn.", cfg, inv_freq, dtype)
        xn = plain_rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = x + plain_swiglu_mlp(
            xn, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"]
        )
    return x


def plain_logits(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], dtype=torch.float32) -> torch.Tensor:
    """Logits at every position of one whole sequence, [T, vocab].

    Final norm then the classifier; a tied model reuses the embedding matrix
    (src/model.rs:1365-1366, :469-473).
    """
    cfg = complete_config(cfg)
    x = plain_hidden(cfg, w, tokens, dtype)
    xn = plain_rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return xn @ head.to(dtype).T


# --------------------------------------------------------------------------- sampling
class PlainRng:
    """xorshift64* of the reference's sampler (src/sampler.rs:176-187); seed 0 becomes 1 (:803)."""

    MASK = (1 << 64) - 1

    def __init__(self, seed: int):
        self.state = (seed & self.MASK) or 1

    def next_u32(self) -> int:
        s = self.state
        s ^= s >> 12
        s ^= (s << 25) & self.MASK
        s ^= s >> 27
        self.state = s
        return ((s * 0x2545F4914F6CDD1D) & self.MASK) >> 32

    def next_f32(self) -> float:
        return float(np.float32(self.next_u32() >> 8) / np.float32(16777216.0))


def plain_argmax(logits: Sequence[float]) -> int:
    """Last of equal maxima; a NaN compares equal, so the element after it
    replaces it (src/sampler.rs:78-84)."""
    best = 0
    for i in range(1, len(logits)):
        a, b = logits[best], logits[i]
        greater = (a > b)  # False when either is NaN
        if not greater:
            best = i
    return best


def _softmax_f32(logits: np.ndarray) -> np.ndarray:
    """Subtract the max, exp, sum in index order, multiply by 1/sum, all in
    32-bit (src/sampler.rs:58-73)."""
    mx = np.float32(-np.inf)
    for v in logits:
        mx = max(mx, v)
    e = np.exp((logits - mx).astype(np.float32)).astype(np.float32)
    total = np.float32(0.0)
    for v in e:
        total = np.float32(total + v)
    inv = np.float32(1.0) / total
    return (e * inv).astype(np.float32)


def plain_sample(logits: Sequence[float], temperature: float, top_p: float, rng: PlainRng) -> int:
    """One token by the reference's default chain (src/sampler.rs:801-819).

    temperature 0: argmax, no draw.  Otherwise logits / t (:101-106); if
    0 < top_p < 1 the nucleus filter (:116-164: softmax, drop p < (1-p)/(n-1),
    sort the rest by p descending, keep the shortest prefix whose mass exceeds
    top_p; nothing survives -> argmax); then the inverse-CDF draw (:190-216)
    with one coin, scaled by the kept mass when a nucleus was cut.
    Equal probabilities keep index order here; the reference's unstable sort
    leaves their order unspecified.
    """
    l = np.asarray(logits, dtype=np.float32)
    n = len(l)
    if temperature == 0.0:
        return plain_argmax(list(l))
    l = (l / np.float32(temperature)).astype(np.float32)
    use_top_p = 0.0 < top_p < 1.0
    if use_top_p:
        p = _softmax_f32(l)
        cutoff = np.float32((np.float32(1.0) - np.float32(top_p)) / np.float32(max(n - 1, 1)))
        kept = [i for i in range(n) if p[i] >= cutoff]
        if not kept:
            ids = [plain_argmax(list(l))]
        else:
            kept.sort(key=lambda i: -float(p[i]))  # stable: ties stay in index order
            cumulative = np.float32(0.0)
            last = len(kept) - 1
            for k, i in enumerate(kept):
                cumulative = np.float32(cumulative + p[i])
                if cumulative > np.float32(top_p):
                    last = k
                    break
            ids = kept[: last + 1]
        coin = np.float32(rng.next_f32())
        mass = np.float32(0.0)
        for i in ids:
            mass = np.float32(mass + p[i])
        target = np.float32(coin * mass)
    else:
        p = _softmax_f32(l)
        ids = list(range(n))
        target = np.float32(rng.next_f32())
    cdf = np.float32(0.0)
    for i in ids:
        cdf = np.float32(cdf + p[i])
        if target < cdf:
            return i
    return ids[-1]


# --------------------------------------------------------------------------- generation
def plain_generate(
    cfg: dict,
    w: Dict[str, torch.Tensor],
    prompt: Sequence[int],
    max_new_tokens: int,
    temperature: float = 0.0,
    top_p: float = 0.9,
    seed: int = 1,
    stop_token_ids: Sequence[int] = (),
    dtype=torch.float32,
    chain: Optional["PlainChain"] = None,
) -> List[int]:
    """Tokens generated after `prompt`, recomputing the whole sequence each step.

    Sample from the last position's logits, stop before emitting a stop token,
    else feed the token back (src/model.rs:1743-1760).  chain: the longer sampler
    chain in the place of the default one.
    """
    rng = PlainRng(seed)
    seq = list(prompt)
    out: List[int] = []
    limit = complete_config(cfg)["max_position_embeddings"]
    while len(out) < max_new_tokens and len(seq) < limit:
        logits = plain_logits(cfg, w, seq, dtype)[-1].to(torch.float32).numpy()
        tok = chain.sample(logits) if chain is not None else plain_sample(logits, temperature, top_p, rng)
        if tok in stop_token_ids:
            break
        out.append(tok)
        seq.append(tok)
    return out


class PlainChain:
    """The reference's longer sampler chain for one sequence: penalties -> top-k -> top-p -> min-p ->
    temperature -> draw, or -> argmax when the temperature is 0 (src/sampler.rs:877-931).  Candidates are
    (id, logit, p) records in an array that the stages reorder and shorten, as in the reference; where it
    sorts with an unstable sort, the stable sort here keeps equal values in index order."""

    def __init__(self, temperature=1.0, top_p=0.9, seed=1, top_k=0, min_p=0.0, repeat_penalty=1.0, repeat_last_n=64,
                 frequency_penalty=0.0, presence_penalty=0.0, mirostat=0, mirostat_lr=0.1, mirostat_ent=5.0, mirostat_m=100,
                 xtc_probability=0.0, xtc_threshold=0.1, dry_multiplier=0.0, dry_base=1.75, dry_allowed_length=2,
                 dry_penalty_last_n=64, dry_sequence_breakers=()):
        self.dry_mult, self.dry_base, self.dry_allowed = dry_multiplier, dry_base, max(dry_allowed_length, 1)
        self.dry_last_n, self.dry_breakers = dry_penalty_last_n, set(dry_sequence_breakers)
        self.dry_ring = []  # DRY's own ring of chosen tokens (src/sampler.rs:735-743)
        self.xtc_p, self.xtc_thr = xtc_probability, xtc_threshold
        self.xtc_rng = PlainRng(seed)  # its own stream from the same seed (src/sampler.rs:547-553)
        self.mirostat, self.eta, self.tau, self.m = mirostat, mirostat_lr, mirostat_ent, mirostat_m
        self.mu = np.float32(2.0) * np.float32(mirostat_ent)  # (src/sampler.rs:379)
        self.t, self.top_p, self.top_k, self.min_p = temperature, top_p, top_k, min_p
        self.repeat, self.last_n, self.freq, self.present = repeat_penalty, repeat_last_n, frequency_penalty, presence_penalty
        self.rng = PlainRng(seed)
        self.ring = []  # the last `last_n` chosen tokens (src/sampler.rs:339-347)

    @staticmethod
    def _softmax(cands):
        """p over the live candidates, 32-bit, in array order (src/sampler.rs:58-73)."""
        l = np.array([c[1] for c in cands], dtype=np.float32)
        p = _softmax_f32(l)
        return [(c[0], c[1], p[k]) for k, c in enumerate(cands)]

    def sample(self, logits) -> int:
        f32 = np.float32
        cands = [(i, f32(v), f32(0.0)) for i, v in enumerate(np.asarray(logits, dtype=np.float32))]
        sorted_by_p = False
        # penalties (src/sampler.rs:314-337)
        penalties_on = self.repeat != 1.0 or self.freq != 0.0 or self.present != 0.0
        if penalties_on and self.ring:
            counts = {}
            for tok in self.ring:
                counts[tok] = counts.get(tok, 0) + 1
            out = []
            for i, l, p in cands:
                if i in counts:
                    l = f32(l / f32(self.repeat)) if l > 0 else f32(l * f32(self.repeat))
                    l = f32(l - f32(counts[i]) * f32(self.freq))
                    l = f32(l - f32(self.present))
                out.append((i, l, p))
            cands = out
        cands = self._dry(cands)
        if self.mirostat:
            return self._accept(self._mirostat(cands))
        # top-k (src/sampler.rs:239-251): the k largest logits; here in descending order
        if self.top_k != 0 and self.top_k < len(cands):
            cands = sorted(cands, key=lambda c: -float(c[1]))[: self.top_k]
        # top-p (src/sampler.rs:120-160)
        if 0.0 < self.top_p < 1.0:
            n = len(cands)
            cands = self._softmax(cands)
            cutoff = f32((f32(1.0) - f32(self.top_p)) / f32(max(n - 1, 1)))
            kept = [c for c in cands if c[2] >= cutoff]
            if not kept:
                best = plain_argmax([float(c[1]) for c in cands])
                cands = [cands[best]]
            else:
                kept.sort(key=lambda c: -float(c[2]))
                cumulative, last = f32(0.0), len(kept) - 1
                for k, c in enumerate(kept):
                    cumulative = f32(cumulative + c[2])
                    if cumulative > f32(self.top_p):
                        last = k
                        break
                cands = kept[: last + 1]
            sorted_by_p = True
        # min-p (src/sampler.rs:265-281)
        if self.min_p > 0.0 and len(cands) >= 2:
            mx = max(float(c[1]) for c in cands)
            thresh = f32(f32(mx) + f32(np.log(f32(self.min_p))))
            cands = sorted(cands, key=lambda c: -float(c[1]))
            above = 0
            for c in cands:
                if c[1] >= thresh:
                    above += 1
                else:
                    break
            cands = cands[: min(max(above, 1), len(cands))]
            sorted_by_p = False
        # XTC (src/sampler.rs:569-602)
        if self.xtc_p > 0.0 and not (self.xtc_thr > 0.5) and len(cands) >= 2:
            chance = f32(self.xtc_rng.next_f32())  # drawn whether or not the filter acts
            if not (chance > f32(self.xtc_p)):
                n = len(cands)
                cands = self._softmax(sorted(cands, key=lambda c: -float(c[1])))
                above = 0
                for c in cands:
                    if c[2] >= f32(self.xtc_thr):
                        above += 1
                    else:
                        break
                pos_last = max(above - 1, 0)
                if pos_last > 0 and n - pos_last >= 1:
                    cands = cands[pos_last:]
                sorted_by_p = True
        if self.t == 0.0:
            sel = plain_argmax([float(c[1]) for c in cands])  # (src/sampler.rs:225-228)
        else:
            cands = [(i, f32(l / f32(self.t)), p) for i, l, p in cands]  # (:101-106), which also drops `sorted`
            sorted_by_p = False
            cands = self._softmax(cands)
            coin = f32(self.rng.next_f32())
            target = coin  # (:199-204: only a sorted array scales the coin)
            cdf, sel = f32(0.0), len(cands) - 1
            for k, c in enumerate(cands):
                cdf = f32(cdf + c[2])
                if target < cdf:
                    sel = k
                    break
        return self._accept(cands[sel][0])

    def _accept(self, token: int) -> int:
        if self.last_n > 0:
            if len(self.ring) == self.last_n:
                self.ring.pop(0)
            self.ring.append(token)
        if self.dry_last_n > 0:
            if len(self.dry_ring) == self.dry_last_n:
                self.dry_ring.pop(0)
            self.dry_ring.append(token)
        return token

    @staticmethod
    def _z_array(s):
        """z[k]: length of the longest common prefix of s and s[k:] (src/sampler.rs:612-635); plainly."""
        n = len(s)
        z = [0] * n
        if n:
            z[0] = n
        for k in range(1, n):
            while k + z[k] < n and s[z[k]] == s[k + z[k]]:
                z[k] += 1
        return z

    def _dry(self, cands):
        """DRY (src/sampler.rs:683-733): the chain holds this stage only when the multiplier is above 0 (:889)."""
        f32 = np.float32
        if not (self.dry_mult > 0.0) or self.dry_base < 1.0 or self.dry_last_n == 0 or len(self.dry_ring) <= self.dry_allowed:
            return cands
        history = list(self.dry_ring)
        n = len(history)
        rep_limit = n
        for i in range(n):
            if history[n - i - 1] in self.dry_breakers:
                rep_limit = i
                break
        if rep_limit <= self.dry_allowed:
            return cands
        rev = history[n - rep_limit:][::-1]
        z = self._z_array(rev)
        max_repeat = {}
        for k in range(1, rep_limit):
            repeat_len = z[k] + 1
            if repeat_len < self.dry_allowed:
                continue
            cont = rev[k - 1]
            max_repeat[cont] = max(max_repeat.get(cont, 0), repeat_len)
        out = []
        for i, l, p in cands:
            if i in max_repeat:
                pw, b, e = f32(1.0), f32(self.dry_base), max_repeat[i] - self.dry_allowed  # powi: by squaring
                while e > 0:
                    if e & 1:
                        pw = f32(pw * b)
                    b = f32(b * b)
                    e >>= 1
                l = f32(l - f32(self.dry_mult) * pw)
            out.append((i, l, p))
        return out

    def _mirostat(self, cands) -> int:
        """penalties (done) -> temperature -> mirostat 1 (src/sampler.rs:401-449) or 2 (:494-524)."""
        f32 = np.float32
        cands = [(i, f32(l / f32(self.t)), p) for i, l, p in cands]
        n = len(cands)
        cands = self._softmax(sorted(cands, key=lambda c: -float(c[1])))
        if self.mirostat == 1:
            bound = min(max(self.m - 1, 0), max(n - 1, 0))
            sum_ti_bi = sum_ti_sq = 0.0
            for i in range(bound):
                t_i = math.log((i + 2) / (i + 1))
                with np.errstate(divide="ignore", invalid="ignore"):
                    b_i = float(np.log(np.float64(cands[i][2]) / np.float64(cands[i + 1][2])))
                sum_ti_bi += t_i * b_i
                sum_ti_sq += t_i * t_i
            with np.errstate(all="ignore"):
                s_hat = np.float64(sum_ti_bi) / np.float64(sum_ti_sq)
                eps = s_hat - 1.0
                k = np.power((eps * np.power(2.0, np.float64(self.mu))) / (1.0 - np.power(-eps, np.float64(n))), 1.0 / s_hat)
            keep = int(k) if np.isfinite(k) and abs(k) < 9.2e18 else (1 if not np.isfinite(k) else (2**63 - 1 if k > 0 else -(2**63)))
            keep = min(max(keep, 1), n)
        else:
            cutoff = n
            for k_, c in enumerate(cands):
                with np.errstate(divide="ignore"):
                    if -np.log2(c[2]) > self.mu:
                        cutoff = k_
                        break
            keep = max(cutoff, 1)
        cands = self._softmax(cands[:keep])
        coin = f32(self.rng.next_f32())
        cdf, sel = f32(0.0), len(cands) - 1
        for k_, c in enumerate(cands):
            cdf = f32(cdf + c[2])
            if coin < cdf:
                sel = k_
                break
        with np.errstate(divide="ignore"):
            observed = f32(-np.log2(cands[sel][2]))
        self.mu = f32(self.mu - f32(self.eta) * f32(observed - f32(self.tau)))
        return cands[sel][0]
