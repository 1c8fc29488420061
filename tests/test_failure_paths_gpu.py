"""Failure paths that need a device but fault nothing: a bounded barrier wait that runs out
reports through the status word and leaves the context usable; guards around the cache's
storage show a write outside it."""
import pytest
import torch

from helpers import make_folder, random_ids

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_sets_the_status_bit_and_returns():
    """The product kernels' own wait helper on a barrier nobody arrives at, with short limits
    (a few thousand tries, 0.2 ms): it gives up, sets bit 4, and the kernel ends normally."""
    from minfer_b200.engine.step import status_bits
    from minfer_b200.kernels import api as K
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    K.wait_probe(status, 1 << 20, 200_000, waited)
    torch.cuda.synchronize()
    assert int(status.item()) == 4
    assert status_bits(4) == ["a bounded wait on a barrier ran out"]
    assert 150_000 <= int(waited.item()) < 50_000_000          # the time limit ended it, soon
    # a limit on the tries alone ends it too
    status.zero_()
    K.wait_probe(status, 2000, 2_000_000_000, waited)
    torch.cuda.synchronize()
    assert int(status.item()) == 4 and int(waited.item()) < 50_000_000
    # the context is as usable as before
    x = torch.randn(3, 64, device="cuda")
    out = torch.empty(3, 64, device="cuda")
    K.rmsnorm(x, torch.ones(64, device="cuda"), 1e-6, out)
    assert torch.isfinite(out).all()


def test_an_engine_reports_a_wait_that_ran_out():
    """The bit in an engine's own status word: ``check_status`` raises and clears it, and the
    next ``step`` raises on its own once the word's copy has arrived on the host."""
    from minfer_b200.engine.step import Engine, StepError
    from minfer_b200.kernels import api as K
    from minfer_b200.model import Model
    eng = Engine(Model.from_folder(make_folder("A"), "bfloat16", "cuda:0"), max_tokens=256)
    s = eng.acquire()
    eng.step([s], [random_ids(9, 256, 1)])
    eng.check_status()
    K.wait_probe(eng.status, 2000, 100_000)
    with pytest.raises(StepError, match="bounded wait on a barrier ran out"):
        eng.check_status()
    eng.check_status()                                          # cleared
    # without anyone calling check_status: the step after the one that carried the word to the
    # host raises
    K.wait_probe(eng.status, 2000, 100_000)
    eng.step([s], [[3]])                                        # launches; posts the word
    torch.cuda.synchronize()
    with pytest.raises(StepError, match="bounded wait on a barrier ran out"):
        eng.step([s], [[4]])
    eng.step([s], [[4]])                                        # and goes on afterwards
    eng.check_status()


def test_guards_around_cache_and_state_show_a_write_outside():
    from minfer_b200.cache.paged import CacheError
    from minfer_b200.engine.generate import Generator
    from minfer_b200.model import Model
    from minfer_b200.sampling.params import SamplingParams
    gen = Generator(Model.from_folder(make_folder("B"), "bfloat16", "cuda:0"), max_tokens=1024,
                    max_batch=4)
    prompts = [random_ids(n, 389, n) for n in (70, 3, 200, 64)]
    gen.generate(prompts, 20, SamplingParams(seed=1), stop_token_ids=[])
    cache = gen.engine.cache
    cache.check_canaries()                                      # all kernels stayed inside
    group = cache.groups[-1]
    guard = group._guarded[1].raw
    guard[guard.numel() - 3] = 0                                # the host plays the stray write
    with pytest.raises(CacheError, match="values of cache group"):
        cache.check_canaries()
    guard[guard.numel() - 3] = 0xA5
    state = cache.state._guarded[0].raw
    state[7] = 1
    with pytest.raises(CacheError, match="state"):
        cache.check_canaries()


def test_generation_stats_hold_device_times():
    from minfer_b200.engine.generate import Generator
    from minfer_b200.model import Model
    from minfer_b200.sampling.params import SamplingParams
    for pipelined in (True, False):
        gen = Generator(Model.from_folder(make_folder("D"), "bfloat16", "cuda:0"), max_tokens=2048,
                        max_batch=2, pipelined=pipelined)
        gen.generate([random_ids(300, 300, 1), random_ids(20, 300, 2), random_ids(5, 300, 3)], 16,
                     SamplingParams.greedy(), stop_token_ids=[])
        st = gen.stats
        assert st.batches == 2
        assert 0.0 < st.prefill_device_seconds < 5.0 and 0.0 < st.decode_device_seconds < 5.0
        # the device cannot have worked longer than the host waited for it
        assert st.prefill_device_seconds + st.decode_device_seconds <= \
            st.prefill_seconds + st.decode_seconds + 0.05
