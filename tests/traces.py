"""Builds the replay traces the tests use: the same requests cut three ways."""
import torch

TAIL = 32


def make_requests(vocab, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lengths)}


def tail_of(tokens):
    return min(TAIL, len(tokens))


def whole(requests):
    """Each request alone and whole, the logits of its last TAIL places wanted."""
    steps = []
    for i, (rid, toks) in enumerate(requests.items()):
        k = tail_of(toks)
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks) - k, len(toks)))}],
                      "end": [rid]})
    return steps


def stepped(requests):
    """Each request alone: all but the last TAIL tokens in one step, then one by one."""
    steps = []
    n = 0
    for rid, toks in requests.items():
        k = tail_of(toks)
        head = len(toks) - k
        if head:
            steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": []}], "end": []})
            n += 1
        for j in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[j]], "want": [0]}],
                          "end": [rid] if j == len(toks) - 1 else []})
            n += 1
    return steps


def batched(requests, batch_size):
    """Batches of unequal lengths that start together: one packed step with every
    request's head, then one token each; a request whose tokens are used up ends
    and leaves the batch; batches follow one another."""
    ids = list(requests)
    steps = []
    n = 0
    for b in range(0, len(ids), batch_size):
        group = ids[b:b + batch_size]
        head = {r: max(1, len(requests[r]) - TAIL) for r in group}
        entries = []
        for r in group:
            toks = requests[r][:head[r]]
            # a request shorter than TAIL+1 starts with one token, whose logits are wanted
            want = [0] if len(requests[r]) <= TAIL else []
            entries.append({"id": r, "tokens": toks, "want": want})
        done = [r for r in group if head[r] == len(requests[r])]
        steps.append({"step": n, "entries": entries, "end": done})
        n += 1
        at = dict(head)
        live = [r for r in group if r not in done]
        while live:
            entries = [{"id": r, "tokens": [requests[r][at[r]]], "want": [0]} for r in live]
            for r in live:
                at[r] += 1
            done = [r for r in live if at[r] == len(requests[r])]
            steps.append({"step": n, "entries": entries, "end": done})
            n += 1
            live = [r for r in live if r not in done]
    return steps


def collect(steps, outputs, vocab):
    """Map (request id, place in the request) -> logits row, from a replay's outputs
    (`outputs[step]` is the [wanted, vocab] array of that step, or None)."""
    at = {}
    rows = {}
    for st in steps:
        out = outputs.get(st["step"])
        k = 0
        for e in st["entries"]:
            base = at.get(e["id"], 0)
            for w in e["want"]:
                rows[(e["id"], base + w)] = out[k]
                k += 1
            at[e["id"]] = base + len(e["tokens"])
        assert out is None or k == out.shape[0]
    return rows


def peak_tokens(steps, page=64):
    """The most tokens live requests hold at any time, each rounded up to whole pages."""
    held, peak = {}, 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-v // page) * page for v in held.values()))
        for r in st["end"]:
            del held[r]
    return peak
