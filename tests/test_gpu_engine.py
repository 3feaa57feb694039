"""The step loop end to end on a small random-init decoder: chunked prefill, continuous batching, page
hand-out and release, CUDA-graph replay.  Graph replay and eager execution run the same kernels on the same
inputs, so their tokens must be identical."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def build(use_graphs, **kw):
    from inference_engine_b200 import scaffold as S
    from inference_engine_b200.engine import Engine

    dev = torch.device("cuda", 0)
    model = S.DecoderScaffold(dev, hidden=256, ffn=512, vocab=1000, layers=2, seed=7)
    args = dict(max_batch_size=4, max_len=512, stop_token_id=-1, max_tokens_per_step=96, min_first_chunk=16,
                max_graph_tokens=96, use_graphs=use_graphs)
    args.update(kw)
    return Engine(model, **args)


def prompts():
    g = torch.Generator().manual_seed(3)
    return [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (5, 150, 33, 70, 16, 201)]


def test_graphs_and_eager_generate_the_same_tokens():
    from inference_engine_b200 import kernels as K

    outs = []
    for use_graphs in (False, True):
        eng = build(use_graphs)
        reqs = eng.generate(prompts(), max_new_tokens=6)
        assert all(len(r.output) == 6 and r.t_finish is not None and r.pages == [] for r in reqs)
        assert eng.sched.idle() and eng.pool.committed == 0 and eng.pool.uncommitted() == eng.pool.capacity
        assert K.check_status() == 0
        if use_graphs:
            assert eng.steps_run["decode_graph"] > 0 and eng.steps_run["mixed_graph"] > 0
        else:
            assert eng.steps_run["eager"] > 0 and eng.steps_run["decode_graph"] == 0
        outs.append([r.output for r in reqs])
    assert outs[0] == outs[1]
    assert all(0 <= t < 1000 for o in outs[0] for t in o)


def test_steps_beyond_the_largest_bucket_run_eagerly_with_the_same_result():
    a = build(True, max_tokens_per_step=96, max_graph_tokens=32)  # buckets 16, 32: most prefill steps are eager
    b = build(True, max_tokens_per_step=96, max_graph_tokens=96)
    ra = a.generate(prompts()[:3], max_new_tokens=4)
    rb = b.generate(prompts()[:3], max_new_tokens=4)
    assert a.steps_run["eager"] > 0
    assert [r.output for r in ra] == [r.output for r in rb]


def test_requests_arriving_while_others_decode():
    eng = build(True)
    p = prompts()
    first = [eng.submit_request(p[1], 8), eng.submit_request(p[2], 8)]
    for _ in range(4):
        eng.step()
    late = eng.submit_request(p[3], 5)
    while not eng.sched.idle():
        eng.step()
    assert [len(r.output) for r in first] == [8, 8] and len(late.output) == 5
    assert late.t_first_token >= first[1].t_first_token
    assert eng.pool.uncommitted() == eng.pool.capacity


def test_sampling_with_temperature_is_reproducible_from_the_seed():
    p = prompts()[:4]
    a = build(True, tau=0.8, seed=11).generate(p, max_new_tokens=5)
    b = build(True, tau=0.8, seed=11).generate(p, max_new_tokens=5)
    c = build(True, tau=0.8, seed=12).generate(p, max_new_tokens=5)
    assert [r.output for r in a] == [r.output for r in b]
    assert [r.output for r in a] != [r.output for r in c]
