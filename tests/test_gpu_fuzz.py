"""Random traffic against the plain implementation: requests of random lengths arrive in
random batches, bring their prompts whole or cut into random chunks, decode token by
token, end at random times, and their slots and pages are used again; every logit that
is asked for is compared.  One tiny configuration with a window, one without."""
import random

import pytest
import torch

from gpu_util import TOL, Oracle, engine, max_err, sharpen
from tiny import make_folder

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name, dtype, seed", [("B", "float32", 0), ("B", "bfloat16", 1), ("C", "float32", 2),
                                               ("C", "bfloat16", 3), ("A", "bfloat16", 4)])
def test_random_traffic(name, dtype, seed, tmp_path):
    folder = sharpen(make_folder(tmp_path, name), 4.0)
    orc = Oracle(folder)
    rng = random.Random(seed)
    g = torch.Generator().manual_seed(seed)
    eng = engine(folder, dtype, max_tokens=64 * 10, max_slots=5, row_multiple=rng.choice([1, 1, 8]))
    live = {}           # slot -> [tokens of the request, how many are in the cache]
    worst, compared = 0.0, 0
    for step in range(140):
        # sometimes start requests (as many as there is room for), sometimes end one
        if len(live) < 5 and rng.random() < 0.35:
            total = rng.choice([1, 2, 3, 17, 63, 64, 65, 100, 150])
            toks = torch.randint(0, orc.cfg.vocab_size, (total,), generator=g).tolist()
            used = sum(-(-len(t) // 64) for t, _ in live.values())
            if used + -(-total // 64) <= 10:
                live[eng.open()] = [toks, 0]
        if live and rng.random() < 0.1:
            s = rng.choice(list(live))
            eng.close(s)
            del live[s]
        ready = [s for s, (t, n) in live.items() if n < len(t)]
        if not ready:
            for s in list(live):
                eng.close(s)
                del live[s]
            continue
        batch = rng.sample(ready, rng.randint(1, len(ready)))
        entries, want, where = [], [], []
        for s in batch:
            toks, n = live[s]
            left = len(toks) - n
            k = 1 if (n > 0 and rng.random() < 0.6) else rng.randint(1, left)       # one token, or a chunk
            w = sorted(rng.sample(range(k), rng.randint(0, min(k, 3))))
            entries.append((s, toks[n:n + k]))
            want.append(w)
            where.append((s, n, w))
            live[s][1] = n + k
        out = eng.step(entries, want=want)
        if out is None:
            continue
        r = 0
        for s, n, w in where:
            ref = orc.logits(live[s][0])
            for i in w:
                worst = max(worst, max_err(out[r], ref[n + i]))
                r += 1
                compared += 1
        for s in list(live):
            if live[s][1] == len(live[s][0]) and rng.random() < 0.5:
                eng.close(s)
                del live[s]
    eng.check()
    assert compared > 60
    assert worst < TOL[dtype], worst
