"""Device-side sample_token against the oracle's restatement of src/generate.rs:698-801.

Penalties, candidate order and the xorshift64 draw are exact on the device; the probabilities can
differ from the CPU's in their last bits (tree-summed softmax denominator, device expf), so the draw
may land on the other side of a boundary in rare cases.  The tests therefore ask for identical tokens
on the overwhelming majority of seeded cases and for exact agreement where no probability is involved
(top_k = 1, peaked logits, RNG state)."""
import numpy as np
import pytest

from homura_b200 import synth

pytestmark = pytest.mark.gpu


def _cfg(hm, **kw):
    base = dict(temperature=0.7, top_k=50, top_p=0.9, min_p=0.0, repetition_penalty=1.1, frequency_penalty=0.0, presence_penalty=0.0)
    base.update(kw)
    return hm.SamplingConfig(**base), base


@pytest.mark.parametrize("kw", [dict(), dict(top_k=1), dict(top_k=1024, top_p=1.0), dict(min_p=0.05, top_p=0.95, temperature=1.3),
                                dict(repetition_penalty=1.0, frequency_penalty=0.4, presence_penalty=0.3), dict(top_k=8, top_p=0.5, repetition_penalty=1.3)])
def test_device_sampler_matches_oracle(hm, oracle, kw):
    cfg, d = _cfg(hm, **kw)
    rng = np.random.default_rng(len(str(kw)))
    V = 32000
    same = total = 0
    for trial in range(40):
        logits = (rng.standard_normal(V) * 3.0).astype(np.float32)
        gen = rng.integers(0, V, size=rng.integers(0, 200)).astype(np.uint32)
        if gen.size:
            gen[: gen.size // 3] = gen[0]  # repeated tokens: the penalties apply per occurrence
        seed = int(rng.integers(1, 2**62)) | 1
        orng = oracle.Rng(seed)
        want = oracle.sample_token(logits, orng, gen, **d)
        got, state = hm.sample_token_device(logits, cfg, gen, seed)
        assert state == int(orng.state.value)  # the integer RNG advances identically
        assert 0 <= got < V
        same += int(got == want)
        total += 1
    assert same >= total - 1, (same, total)
    if d["top_k"] == 1:
        assert same == total


def test_device_sampler_ties_and_peaks(hm, oracle):
    cfg, d = _cfg(hm, top_k=4, top_p=1.0, repetition_penalty=1.0)
    V = 1000
    # one dominant logit: probability 1 up to rounding, always chosen
    logits = np.full(V, -30.0, np.float32)
    logits[777] = 20.0
    for seed in (1, 3, 12345):
        assert hm.sample_token_device(logits, cfg, [], seed)[0] == 777
    # all equal: the candidates are the four lowest indices (ties resolve by index) with probability 1/V each
    flat = np.zeros(V, np.float32)
    seen = {hm.sample_token_device(flat, cfg, [], ((s * 0x9E3779B97F4A7C15) & (2**64 - 1)) | 1)[0] for s in range(1, 100)}  # well-mixed seeds
    assert seen == {0, 1, 2, 3}
    # the same at a vocabulary with far more ties at the cut than the candidate list holds: still the lowest indices
    flat = np.zeros(32000, np.float32)
    seen = {hm.sample_token_device(flat, cfg, [], ((s * 0x9E3779B97F4A7C15) & (2**64 - 1)) | 1)[0] for s in range(1, 100)}
    assert seen == {0, 1, 2, 3}
    # rows masked to -inf with fewer finite entries than top_k: the finite ones first, then the lowest masked indices
    masked = np.full(32000, -np.inf, np.float32)
    masked[[9000, 17]] = [2.0, 1.0]
    cfg8, _ = _cfg(hm, top_k=8, top_p=1.0, repetition_penalty=1.0)
    seen = {hm.sample_token_device(masked, cfg8, [], ((s * 0x9E3779B97F4A7C15) & (2**64 - 1)) | 1)[0] for s in range(1, 60)}
    assert seen <= {9000, 17} and 9000 in seen


def test_greedy_with_penalties_on_device(hm, oracle):
    # the reference CLI's `--temperature 0` keeps the default repetition penalty 1.1 (src/generate.rs:676,707-745):
    # penalties, then argmax with ties to the highest index; the RNG is not touched
    rng = np.random.default_rng(3)
    V = 151936
    for trial, kw in enumerate([dict(repetition_penalty=1.1), dict(repetition_penalty=1.3, frequency_penalty=0.5, presence_penalty=0.2), dict(repetition_penalty=1.0, presence_penalty=4.0)]):
        cfg, d = _cfg(hm, temperature=0.0, top_k=50, **kw)
        logits = rng.standard_normal(V).astype(np.float32)
        top = np.argsort(logits)[-6:]
        gen = np.concatenate([top[-3:], top[-1:], rng.integers(0, V, size=50)]).astype(np.uint32)  # the leaders were generated before
        logits[top[-2]] = logits[top[-1]]  # and two of them tie
        orng = oracle.Rng(99)
        want = oracle.sample_token(logits, orng, gen, **d)
        got, state = hm.sample_token_device(logits, cfg, gen, 99)
        assert got == want and state == 99
        assert got == hm.sample_token(logits, cfg, gen, 99)[0]
    # ties resolve to the highest index
    flat = np.zeros(V, np.float32)
    cfg, _ = _cfg(hm, temperature=0.0, repetition_penalty=1.1)
    assert hm.sample_token_device(flat, cfg, [V - 1], 1)[0] == V - 1  # 0 * 1.1 is still 0: every entry ties
    assert hm.sample_token_device(flat, hm.SamplingConfig(temperature=0.0, repetition_penalty=1.0, presence_penalty=1.0), [V - 1], 1)[0] == V - 2


def test_top_k_disabled_or_wide_on_device(hm, oracle):
    # top_k = 0 ("disabled", src/generate.rs:652) and top_k above the 1024 candidates the kernel gathers: exact
    # while the top-p prefix ends inside the candidates; otherwise the host sampler finishes the token
    rng = np.random.default_rng(8)
    V = 32000
    for top_k in (0, 5000, V):
        cfg, d = _cfg(hm, top_k=top_k, top_p=0.9, repetition_penalty=1.1)
        same = 0
        for trial in range(20):
            logits = (rng.standard_normal(V) * 4.0).astype(np.float32)  # peaked: 0.9 of the mass within a few hundred tokens
            gen = rng.integers(0, V, size=30).astype(np.uint32)
            seed = int(rng.integers(1, 2**62)) | 1
            orng = oracle.Rng(seed)
            want = oracle.sample_token(logits, orng, gen, **d)
            got, state = hm.sample_token_device(logits, cfg, gen, seed)
            assert state == int(orng.state.value)
            same += int(got == want)
        assert same >= 19, (top_k, same)
    # nearly flat row, top-p 0.9 spans most of the vocabulary: handed to the host sampler, bit-identical to it
    cfg, d = _cfg(hm, top_k=0, top_p=0.9, repetition_penalty=1.0)
    for trial in range(5):
        logits = (rng.standard_normal(V) * 0.01).astype(np.float32)
        seed = int(rng.integers(1, 2**62)) | 1
        assert hm.sample_token_device(logits, cfg, [], seed) == hm.sample_token(logits, cfg, [], seed)


@pytest.mark.parametrize("vocab", [1024, 20000])
def test_batched_sampled_decode_step(hm, oracle, vocab):
    # hm_decode_step_sampled: decode_step + sample_token for every sequence of a batch, one RNG word each.  The small
    # vocabulary runs the one-CTA kernel, the large one a cluster of eight CTAs per sequence.
    import tempfile

    cfg = synth.tiny_config(vocab_size=vocab)
    d = synth.write_hf_model(tempfile.mkdtemp(), cfg, seed=7, norm_jitter=0.1)
    B = 3
    m = hm.HfModel.load(d)
    m.init_kv_cache(96, batch=B)
    oms = [oracle.OracleModel.from_hf_dir(d, max_seq_len=96) for _ in range(B)]
    sc = hm.SamplingConfig(temperature=0.8, top_k=40, top_p=0.9, repetition_penalty=1.2, frequency_penalty=0.1, seed=None)
    kw = dict(temperature=0.8, top_k=40, top_p=0.9, min_p=0.0, repetition_penalty=1.2, frequency_penalty=0.1, presence_penalty=0.0)
    states = np.array([(1000 + 17 * b) | 1 for b in range(B)], np.uint64)
    orngs = [oracle.Rng(int(states[b])) for b in range(B)]
    cur, gens = [], []
    for b in range(B):
        ids = synth.prompt_ids(70 + b, 6 + 2 * b, cfg.vocab_size)
        t_o, _ = oms[b].prefill(ids)
        assert m.prefill(ids, seq=b) == t_o
        cur.append(t_o)
        gens.append([t_o])
    same = total = 0
    for step in range(24):
        lg, nxt = m.decode_step_sampled(cur, sc, states, want_logits=True)
        for b in range(B):
            lo = oms[b].decode_step(cur[b])
            assert float(np.abs(lg[b] - lo).max()) <= 1e-4 * max(1.0, float(np.abs(lo).max()))
            want = oracle.sample_token(lo, orngs[b], gens[b], **kw)
            assert int(states[b]) == int(orngs[b].state.value)
            same += int(int(nxt[b]) == want)
            total += 1
            # both sides continue with the oracle's token, so one near-boundary draw cannot derail the rest
            cur[b] = want
            gens[b].append(want)
    assert same >= total - 2, (same, total)
    # greedy with the reference's default penalty, batched: identical to the oracle (no probabilities involved)
    g = hm.SamplingConfig(temperature=0.0, repetition_penalty=1.1)
    gkw = dict(kw, temperature=0.0, repetition_penalty=1.1, frequency_penalty=0.0)
    for step in range(12):
        _, nxt = m.decode_step_sampled(cur, g, states)
        for b in range(B):
            lo = oms[b].decode_step(cur[b])
            want = oracle.sample_token(lo, orngs[b], gens[b], **gkw)
            assert int(nxt[b]) == want
            cur[b] = want
            gens[b].append(want)
    m.close()


def test_sampled_generation_on_device(hm, oracle, monkeypatch):
    import tempfile

    cfg = synth.tiny_config()
    d = synth.write_hf_model(tempfile.mkdtemp(), cfg, seed=7, norm_jitter=0.1)
    ids = synth.prompt_ids(5, 12, cfg.vocab_size)
    m = hm.HfModel.load(d)
    m.init_kv_cache(128)
    sc = hm.SamplingConfig(temperature=0.8, top_k=40, top_p=0.9, repetition_penalty=1.1, seed=1234)
    dev = m.generate_ids(ids, 48, sc)
    assert len(dev) == 48 and all(0 <= t < cfg.vocab_size for t in dev) and m.kv_cache_len() == 12 + 47
    # reproducible for a seed, and top_k = 1 is greedy decoding whatever the temperature
    m.reset_kv_cache()
    assert m.generate_ids(ids, 48, sc) == dev
    m.reset_kv_cache()
    greedy = m.generate_ids(ids, 24, hm.SamplingConfig.greedy())
    m.reset_kv_cache()
    assert m.generate_ids(ids, 24, hm.SamplingConfig(temperature=0.8, top_k=1, top_p=1.0, repetition_penalty=1.0, seed=5)) == greedy
    # the reference CLI's greedy mode (temperature 0, repetition penalty 1.1) stays on the device and differs from plain argmax decoding
    m.reset_kv_cache()
    cli = m.generate_ids(ids, 40, hm.SamplingConfig(temperature=0.0))
    m.reset_kv_cache()
    wide = m.generate_ids(ids, 24, hm.SamplingConfig(temperature=0.8, top_k=0, top_p=0.9, repetition_penalty=1.1, seed=1234))
    assert len(cli) == 40 and len(wide) == 24
    # the host sampler on the same seed walks the same candidates: the sequences agree (tiny vocabulary, wide gaps)
    m.close()
    monkeypatch.setenv("HM_HOST_SAMPLER", "1")
    m2 = hm.HfModel.load(d)
    m2.init_kv_cache(128)
    host = m2.generate_ids(ids, 48, sc)
    agree = sum(int(a == b) for a, b in zip(dev, host))
    assert host[:8] == dev[:8] and agree >= 40, (agree, dev, host)
    m2.reset_kv_cache()
    assert m2.generate_ids(ids, 40, hm.SamplingConfig(temperature=0.0)) == cli  # penalties + argmax: no probabilities, so exactly equal
    m2.reset_kv_cache()
    host_wide = m2.generate_ids(ids, 24, hm.SamplingConfig(temperature=0.8, top_k=0, top_p=0.9, repetition_penalty=1.1, seed=1234))
    assert host_wide[:6] == wide[:6]
