"""CPU restatement of the reference's sampler (go/model/sample.go), pure Python over NumPy scalars.

THIS FILE IS TEST INFRASTRUCTURE (the checker for the library's sampler), never imported by the
shipped package. Each function cites the lines it follows. float32 arithmetic is kept in the
reference's operation order with np.float32 scalars; exp runs in float64 as math.Exp does.
Parity status: pinned to the source text and to the closed-form checks in tests/test_sampler_cpu.py
(the splitmix64 stream's first values, the top-k-first / full-path equivalence the reference itself
argues at sample.go:165-175); the reference holds no golden token sequences for it."""
import math

import numpy as np

F = np.float32


def bf16_to_f32(bits) -> np.float32:
    return np.array([int(bits) << 16], dtype=np.uint32).view(np.float32)[0]


def f32_to_bf16(v) -> int:
    """f32ToBF16 (sample.go:510-513): round to nearest even on the bit pattern."""
    b = int(np.array([v], dtype=np.float32).view(np.uint32)[0])
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16) & 0xFFFF


class SampleParams:
    def __init__(self, temperature=0.0, top_k=0, top_p=0.0, min_p=0.0, suppress=(), min_tokens_before_stop=0, repeat_penalty=0.0):
        self.temperature, self.top_k, self.top_p, self.min_p = F(temperature), int(top_k), F(top_p), F(min_p)
        self.suppress, self.min_tokens_before_stop, self.repeat_penalty = list(suppress), int(min_tokens_before_stop), F(repeat_penalty)


class Sampler:
    """model.Sampler (sample.go:64-104)."""

    def __init__(self, seed: int):
        self.state = seed & 0xFFFFFFFFFFFFFFFF

    def next(self) -> np.float32:  # sample.go:97-104
        m = 0xFFFFFFFFFFFFFFFF
        self.state = (self.state + 0x9E3779B97F4A7C15) & m
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
        z ^= z >> 31
        return F(z >> 40) / F(1 << 24)

    def sample(self, logits_bits, p: SampleParams, ids=None) -> int:
        """sampleMapped (sample.go:141-224). logits_bits: bf16 bit patterns; ids: candidate ids or None."""
        vocab = len(logits_bits)
        vals32 = (np.asarray(logits_bits, dtype=np.uint32) << 16).view(np.float32)
        idof = (lambda i: int(ids[i])) if ids is not None else (lambda i: i)
        sup = set(p.suppress)

        def top1():  # greedySuppressed / topMappedSuppressed (sample.go:410-447): strict '>', first wins
            best, bv = -1, F(-np.inf)
            for i in range(vocab):
                if idof(i) in sup:
                    continue
                if vals32[i] > bv:
                    best, bv = i, vals32[i]
            if best < 0:
                raise ValueError("all tokens are suppressed")
            return idof(best)

        if p.temperature <= 0 and p.min_p <= 0:
            return top1()
        if p.top_k == 1:
            t = top1()
            self.next()
            return t
        temp = p.temperature if p.temperature > 0 else F(1)
        rank_filter = (0 < p.top_k < vocab) or (0 < p.top_p < 1) or p.min_p > 0  # sample.go:329-337
        if rank_filter and 0 < p.top_k < vocab:
            return self._topk_first(vals32, idof, sup, vocab, temp, p)
        max_l, allowed = F(-np.inf), 0
        for i in range(vocab):
            if idof(i) in sup:
                continue
            v = vals32[i] / temp
            allowed += 1
            if v > max_l:
                max_l = v
        if allowed == 0:
            raise ValueError("all tokens are suppressed")
        probs = np.zeros(vocab, dtype=np.float32)
        s = F(0)
        for i in range(vocab):
            if idof(i) in sup:
                continue
            v = vals32[i] / temp
            e = F(math.exp(float(v - max_l)))
            probs[i] = e
            s = F(s + e)
        if not rank_filter:  # sampleMappedInVocabOrder (sample.go:379-404)
            if s == 0:
                raise ValueError("empty sampled distribution")
            target = F(self.next() * s)
            acc = F(0)
            for i in range(vocab):
                acc = F(acc + probs[i])
                if acc >= target:
                    return idof(i)
            return idof(vocab - 1)
        order = sorted(range(vocab), key=lambda i: -float(probs[i]))  # stable descending (sort.SliceStable)
        return self._draw_from_ranked(order, probs, idof, vocab, vocab, s, p)

    def _topk_first(self, vals32, idof, sup, vocab, temp, p):  # sample.go:230-262
        vals = np.empty(vocab, dtype=np.float32)
        allowed = 0
        for i in range(vocab):
            if idof(i) in sup:
                vals[i] = F(-np.inf)
                continue
            vals[i] = vals32[i] / temp
            allowed += 1
        if allowed == 0:
            raise ValueError("all tokens are suppressed")
        keep = min(p.top_k, vocab)
        # selectTopKDesc (sample.go:339-366): the first keep of a stable descending sort, ties by ascending index
        order = sorted(range(vocab), key=lambda i: (-float(vals[i]), i))[:keep]
        max_l = vals[order[0]]
        for i in order:
            vals[i] = F(math.exp(float(vals[i] - max_l)))
        return self._draw_from_ranked(order, vals, idof, keep, vocab, F(0), p)

    def _draw_from_ranked(self, order, probs, idof, keep, vocab, total, p):  # sample.go:271-327
        if 0 < p.top_p < 1:
            kept = total
            if keep != vocab:
                kept = F(0)
                for i in range(keep):
                    kept = F(kept + probs[order[i]])
            cum, n = F(0), 0
            while n < keep:
                cum = F(cum + probs[order[n]])
                n += 1
                if cum >= F(p.top_p * kept):
                    break
            keep = n
        if p.min_p > 0 and keep > 0:
            thr = F(probs[order[0]] * p.min_p)
            n = 0
            while n < keep and probs[order[n]] >= thr:
                n += 1
            if n > 0:
                keep = n
        ksum = F(0)
        for i in range(keep):
            ksum = F(ksum + probs[order[i]])
        target = F(self.next() * ksum)
        acc = F(0)
        for i in range(keep):
            acc = F(acc + probs[order[i]])
            if acc >= target:
                return idof(order[i])
        return idof(order[keep - 1])


def apply_repeat_penalty(logits_bits, history, penalty):
    """applyRepeatPenaltyBF16Into (sample.go:469-508): returns a penalised copy of the bf16 row."""
    out = np.array(logits_bits, dtype=np.uint16, copy=True)
    if penalty <= 1 or len(history) == 0:
        return out
    for tid in sorted(set(int(h) for h in history if 0 <= int(h) < len(out))):
        v = bf16_to_f32(out[tid])
        v = F(v / F(penalty)) if v > 0 else F(v * F(penalty))
        out[tid] = f32_to_bf16(v)
    return out


def generate_sampled(step_logits_bits, sampler: Sampler, p: SampleParams, max_new, stop=()):
    """The decode loop of model/token.go:263-305 with the pick of :361-371: step_logits_bits(token or
    None) returns the bf16 row after feeding the previous pick (None: the prompt's row)."""
    gen, history, stop = [], [], list(stop)
    prev = None
    while len(gen) < max_new:
        row = step_logits_bits(prev)
        if p.repeat_penalty > 1:
            row = apply_repeat_penalty(row, history, p.repeat_penalty)
        pp = p
        if p.min_tokens_before_stop > 0 and len(gen) < p.min_tokens_before_stop:
            pp = SampleParams(p.temperature, p.top_k, p.top_p, p.min_p, list(p.suppress) + [t for t in stop if t not in p.suppress],
                              p.min_tokens_before_stop, p.repeat_penalty)
        nxt = sampler.sample(row, pp)
        gen.append(nxt)
        if p.repeat_penalty > 1:
            history.append(nxt)
        if nxt in stop or len(gen) >= max_new:
            break
        prev = nxt
    return gen
