"""Host-visible failure behaviour and several engines in one process.

* Every device-side wait of the library is bounded; one that runs out raises the engine's device error word
  and the pass that saw it returns HM_ERR_TIMEOUT.  The test makes a wait run out the harmless way: a
  one-CTA probe kernel whose mbarrier is armed for bytes nobody sends (hm_selftest_expire_wait) -- nothing
  faults, traps or hangs, and the next call on the engine is clean.
* Homura is one process (src/hf/model.rs:17-31): a host with several GPUs creates one engine per GPU and
  drives each from its own thread.  Kernel attributes (shared-memory limit, cluster size) are per device, so
  the second engine must set its own.  Runs only where two GPUs are visible."""
import tempfile
import threading

import numpy as np
import pytest

from homura_b200 import synth

pytestmark = pytest.mark.gpu


def _model(seed=7):
    cfg = synth.tiny_config()
    d = synth.write_hf_model(tempfile.mkdtemp(), cfg, seed=seed, norm_jitter=0.1)
    return cfg, d


def test_expired_wait_is_reported_once_and_the_engine_stays_usable(hm):
    cfg, d = _model()
    m = hm.HfModel.load(d)
    m.init_kv_cache(64)
    ids = synth.prompt_ids(3, 12, cfg.vocab_size)
    first = m.prefill(ids)
    _, nxt = m.decode_step([first], want_logits=False)
    clean = int(nxt[0])
    # per-token call
    m.selftest_expire_wait()
    with pytest.raises(hm.HomuraError) as e:
        m.decode_step([clean], want_logits=False)
    assert e.value.status == hm.HM_ERR_TIMEOUT and "bounded" in e.value.message
    # the engine answers again; same tokens as an undisturbed run
    m.reset_kv_cache()
    assert m.prefill(ids) == first
    _, nxt = m.decode_step([first], want_logits=False)
    assert int(nxt[0]) == clean
    # the on-device loop and prefill report it too
    m.selftest_expire_wait()
    with pytest.raises(hm.HomuraError) as e:
        m.decode_greedy_n([clean], 4)
    assert e.value.status == hm.HM_ERR_TIMEOUT
    m.reset_kv_cache()
    m.selftest_expire_wait()
    with pytest.raises(hm.HomuraError) as e:
        m.prefill(ids)
    assert e.value.status == hm.HM_ERR_TIMEOUT
    m.reset_kv_cache()
    assert m.generate_ids(ids, 8, hm.SamplingConfig.greedy())[0] == first
    m.close()


def test_two_engines_on_two_gpus_from_two_threads(hm, oracle):
    if hm.device_count() < 2:
        pytest.skip("needs two GPUs")
    cfg, d = _model(seed=9)
    ids = synth.prompt_ids(5, 20, cfg.vocab_size)
    want = oracle.OracleModel.from_hf_dir(d, max_seq_len=96).generate_greedy(ids, 32)
    out, err = {}, {}

    def run(dev):
        try:
            m = hm.HfModel.load(d, device=dev)
            m.init_kv_cache(96, batch=1)
            a = m.generate_ids(ids, 32, hm.SamplingConfig.greedy())
            # a second model on the same device, with a batch that takes the tensor-core path and other kernels
            m2 = hm.HfModel.load(d, device=dev)
            m2.init_kv_cache(96, batch=12)
            firsts = [m2.prefill(ids, seq=b) for b in range(12)]
            toks = m2.decode_greedy_n(firsts, 8)
            out[dev] = (a, firsts, toks.tolist())
            m.close()
            m2.close()
        except Exception as ex:  # surfaced in the main thread
            err[dev] = ex

    # device 1 first, alone: nothing device 0 set up earlier in this process may be assumed there
    t1 = threading.Thread(target=run, args=(1,))
    t1.start()
    t1.join()
    assert not err, err
    ts = [threading.Thread(target=run, args=(dev,)) for dev in (0, 1)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert not err, err
    for dev in (0, 1):
        a, firsts, toks = out[dev]
        assert a == want
        assert firsts == [want[0]] * 12
        assert all(row == want[1:9] for row in toks)
