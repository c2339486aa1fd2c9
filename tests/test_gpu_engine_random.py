"""Random engine settings, arrivals, cancellations and stop tokens: whatever
the scheduler makes of them (portions, mixed steps, preemption, graphs or none,
overlapped steps or none), every request's tokens are the plain
implementation's greedy choice, every request ends for the right reason, and
every page comes back."""
import numpy as np
import pytest

import plain_hunyuan as ph
import tiny_configs

pytestmark = pytest.mark.gpu


def one_trial(seed, model_folders, many=False):
    """``many``: up to 40 requests under a limit of up to 40 (decode buckets above 16, limits that are
    no power of two), pages of 8 to 256 tokens, the layer sizes of a real model among the configurations."""
    from crane_b200.generation import ModelForCausalLM
    from crane_b200.sampling.sampler import SamplingParams
    rng = np.random.default_rng(seed)
    name = str(rng.choice(["A", "B", "C", "S18", "S18"] if many else ["A", "B", "C"]))
    dt = str(rng.choice(["float32", "bfloat16"]))
    folder = model_folders(name, dt)
    pc, pw = ph.load_folder(folder)
    ps = int(rng.choice([8, 16, 32, 64, 128, 256] if many else [16, 32, 64]))
    n_req = int(rng.integers(2, 41 if many else 9))
    longest = min(100, pc.max_position_embeddings - 45)
    prompts = [rng.integers(0, pc.vocab_size, int(rng.integers(1, longest))).tolist() for _ in range(n_req)]
    new = [int(rng.integers(1, 25 if many else 40)) for _ in range(n_req)]
    need = max(-(-(len(p) + n) // ps) for p, n in zip(prompts, new))       # pages of the largest request
    pages = int(need + rng.integers(0, 3 * need + 2))
    opts = dict(page_size=ps, num_pages=pages, max_concurrent=int(rng.integers(1, 41 if many else 6)),
                max_batched_tokens=int(rng.choice([8, 16, 33, 64, 128])),
                chunk_size=int(rng.choice([4, 8, 32, 64, 2048])),
                use_cuda_graphs=bool(rng.random() < 0.7), async_scheduling=bool(rng.random() < 0.7),
                mixed_decode_min_keys=int(rng.choice([0, 2048])))
    opts["max_batched_tokens"] = max(opts["max_batched_tokens"], opts["max_concurrent"])
    label = f"seed {seed}: {name} {dt} {opts} prompts {[len(p) for p in prompts]} new {new}"
    m = ModelForCausalLM.from_pretrained(folder, dt, **opts)
    eng = m.engine
    arrive = sorted(int(rng.integers(0, 30)) for _ in range(n_req))
    cancel_at = {j: int(rng.integers(1, 40)) for j in range(n_req) if rng.random() < 0.15}
    stop = {}
    for j, p in enumerate(prompts):
        if rng.random() < 0.3 and new[j] > 3:
            full = ph.greedy_generate(pc, pw, p, new[j])
            stop[j] = full[len(p) + int(rng.integers(1, new[j]))]
    ids, step, nxt = {}, 0, 0
    while nxt < n_req or eng.has_work():
        while nxt < n_req and arrive[nxt] <= step:
            ids[nxt] = eng.add_request(prompts[nxt], SamplingParams(), new[nxt], [stop.get(nxt, -1)])
            nxt += 1
        eng.step()
        step += 1
        for j, at in cancel_at.items():
            if at == step and j in ids:
                eng.cancel(ids[j])
        assert step < 5000, label
    m.runner.rt.check_errors()
    m.runner.table.check()
    assert m.runner.table.free_pages() == pages and m.runner.table.live() == 0, label
    tol = 1e-4 if dt == "float32" else 3e-2
    for j, p in enumerate(prompts):
        out = eng.finished[ids[j]]
        got = out.tokens
        assert got[:len(p)] == p, label
        if out.finish_reason == "cancelled":
            assert j in cancel_at, label
        elif out.finish_reason == "stop":
            assert j in stop and got[-1] == stop[j] and stop[j] not in got[len(p):-1], (label, j)
        else:
            assert out.finish_reason == "length" and len(got) == len(p) + new[j], (label, j, out.finish_reason)
        if len(got) > len(p):
            logits = ph.logits_all(pc, pw, got[:-1])
            for t in range(len(p), len(got)):
                row = logits[t - 1]
                assert row[got[t]] >= row.max() - tol * np.abs(row).max(), (label, j, t, got[t], int(row.argmax()))
    return eng.stats()["preemptions"]


def test_random_settings_arrivals_cancellations_and_stop_tokens(model_folders):
    preemptions = sum(one_trial(1000 + i, model_folders) for i in range(24))
    assert preemptions > 0            # some of the pools were small enough to run out


def test_many_requests_under_limits_that_are_no_power_of_two(model_folders):
    for i in range(8):
        one_trial(2000 + i, model_folders, many=True)
