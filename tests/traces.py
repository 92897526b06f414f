"""Builders of replay traces: the same requests cut into steps in different ways.

A trace is a list of steps ``{"step", "entries": [{"id", "tokens", "want"}],
"end"}``; ``peak_tokens`` says how many tokens live requests hold at most, each
rounded up to a multiple of 64, which is what the cache pool is sized for."""
import random


def whole(requests):
    """Each request alone, all of it in one step, every position wanted."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [
            {"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}], "end": [rid]})
    return steps


def tail_decode(requests, tail=32):
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [
            {"id": rid, "tokens": list(toks[:head]), "want": list(range(head))}], "end": []})
        for i in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [
                {"id": rid, "tokens": [toks[i]], "want": [0]}], "end": []})
        steps[-1]["end"] = [rid]
    return steps


def portions(requests, sizes=(5, 2, 9, 3, 2, 17, 1, 4, 31, 2)):
    """Portions of changing size, down to two tokens (and single ones)."""
    steps = []
    k = 0
    for rid, toks in requests.items():
        i = 0
        while i < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - i)
            k += 1
            steps.append({"step": len(steps), "entries": [
                {"id": rid, "tokens": list(toks[i:i + n]), "want": list(range(n))}], "end": []})
            i += n
        steps[-1]["end"] = [rid]
    return steps


def mixed(requests, max_live=4, seed=0, decode_tail=12):
    """Up to ``max_live`` requests at once: portions of some prompts beside single
    tokens of others, requests sitting out steps, finished requests replaced by
    new ones so that their pages are used again."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live = {}      # rid -> [tokens, fed]
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = [list(toks), 0]
        entries, ended = [], []
        for rid in list(live):
            toks, fed = live[rid]
            if len(live) > 1 and rng.random() < 0.25:
                continue                        # sits this step out
            left = len(toks) - fed
            if left <= decode_tail:
                n = 1                           # decoding: one token
            else:
                n = min(left - decode_tail, rng.choice([2, 3, 5, 8, 13, 21]))
            want = list(range(n)) if rng.random() < 0.8 else [n - 1]
            entries.append({"id": rid, "tokens": toks[fed:fed + n], "want": want})
            live[rid][1] = fed + n
            if fed + n == len(toks):
                ended.append(rid)
                del live[rid]
        if not entries:
            continue
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def peak_tokens(steps):
    """Most tokens held by live requests at any time, each rounded up to 64."""
    held, peak = {}, 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // 64) * 64 for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


def collect(steps, outputs):
    """{(request id, position): logits row} from per-step outputs (a list aligned
    with ``steps`` holding [wanted, vocab] arrays or None)."""
    pos = {}
    rows = {}
    for st, out in zip(steps, outputs):
        r = 0
        for e in st["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                rows[(e["id"], base + w)] = out[r]
                r += 1
            pos[e["id"]] = base + len(e["tokens"])
        assert out is None or r == len(out)
    return rows
