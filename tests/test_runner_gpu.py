"""The device-resident generation loop unmasks exactly the tokens the host-driven loop does (which builds
each step's Context the way the reference's ModelRunner.prepare_full / prepare_sparse do)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_device_state_generation_equals_host_driven_generation(cuda_device):
    from dyllm_b200 import _lib, runner
    from dyllm_b200.model import LLaDAForDLM, LLaDAShape, init_weights_

    shape = LLaDAShape(hidden_size=256, num_attention_heads=2, n_kv_heads=2, head_dim=128, mlp_hidden_size=512,
                       num_hidden_layers=3, vocab_size=1024, mask_token_id=1000, max_sequence_length=256)
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(cuda_device):
            model = LLaDAForDLM(shape, 0.99)
    finally:
        torch.set_default_dtype(torch.float32)
    init_weights_(model, seed=3, std=0.05)
    model.eval()
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, 900, (3, 40), generator=g).tolist()
    sr = runner.StepRunner(model, shape.mask_token_id, block_length=8, steps=32, num_full_steps=4, refresh_period=4,
                           use_graphs=False)
    host = sr.generate(prompts, 32, device_state=False)
    dev = sr.generate(prompts, 32, device_state=True)
    assert _lib.load().dyllm_device_status() == 0
    assert host == dev
    assert all(t != shape.mask_token_id for row in dev for t in row)
    # deterministic across runs
    assert sr.generate(prompts, 32, device_state=True) == dev

    # captured steps (CUDA graphs) replay the same launches: first generation warms and captures, the
    # second one is replay only; launches are still accounted for
    gr = runner.StepRunner(model, shape.mask_token_id, block_length=8, steps=32, num_full_steps=4, refresh_period=4,
                           use_graphs=True)
    first = gr.generate(prompts, 32)
    assert len(gr._graphs) == 3
    before = _lib.launch_count
    second = gr.generate(prompts, 32)
    assert _lib.launch_count > before
    assert _lib.load().dyllm_device_status() == 0
    assert first == dev and second == dev
    other = torch.randint(0, 900, (3, 40), generator=g).tolist()
    assert gr.generate(other, 32) == sr.generate(other, 32, device_state=True)


_SEGMENT_SCRIPT = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.getcwd())
torch.cuda.set_device(0)
dist.init_process_group("nccl", init_method="tcp://127.0.0.1:%d" % int(sys.argv[1]), rank=0, world_size=1,
                        device_id=torch.device("cuda:0"))
from dyllm_b200 import layers, runner
x = torch.arange(8, dtype=torch.float32, device="cuda")
out = torch.zeros(8, device="cuda")
def step():
    a = x * 2
    layers.all_reduce_sum(a)      # world size 1: identity, but it cuts the capture
    b = a + 1
    layers.all_reduce_sum(b)
    out.copy_(b * 3)
seg = runner._SegmentedCapture(torch.cuda.graph_pool_handle())
seg.capture(step)
kinds = [k for k, _ in seg.items]
assert kinds == ["graph", "reduce", "graph", "reduce", "graph"], kinds
for scale in (1.0, 5.0):
    x.copy_(torch.arange(8, dtype=torch.float32) * scale)
    seg.replay()
    torch.cuda.synchronize()
    assert torch.equal(out.cpu(), (torch.arange(8, dtype=torch.float32) * scale * 2 + 1) * 3)
assert layers._all_reduce_hook is None
dist.destroy_process_group()
print("segments ok")
"""


def test_segmented_capture_cuts_graphs_at_collectives(cuda_device, tmp_path):
    """A step with collectives is captured as graph / all-reduce / graph ...; replay follows new inputs."""
    import os
    import socket
    import subprocess
    import sys

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = tmp_path / "segments.py"
    script.write_text(_SEGMENT_SCRIPT)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, str(script), str(port)], cwd=root, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "segments ok" in res.stdout, res.stdout + res.stderr


def test_token_ids_follow_the_reference_step_loop(cuda_device):
    """Token ids over a fixed step count against the reference's own step loop (fixture
    tests/golden/llada_tokens_small.pt from tests/golden/make_token_golden.py: the reference's ModelRunner
    preparation, LLaDAForDLM and sampler on the CPU).  Every step is compared and then the recorded choice is
    applied, so one rounding-dependent choice cannot derail the steps after it.  Per step:

    * every candidate row's confidence is within 25 % of the reference's (mean error of a step within 8 %): with
      random-init weights the vocabulary projection turns the ~0.5 % bf16 noise of the hidden states into a few
      per cent of confidence, and the candidates of a block lie only a few per cent apart;
    * a candidate's best token is the reference's wherever that token leads its runner-up by 50 % (two
      probabilities that each move by up to ~14 % can swap a 30 % lead);
    * the rows chosen for unmasking are the reference's wherever the last chosen confidence leads the first
      rejected one by 25 %;
    * every layer's salient set equals the reference's on all rows whose reference cosine is at least 2e-3 from
      the threshold.  The first decision inside that band that goes the other way forks the two runs (the row's
      FFN output is fresh in one and cached in the other), after which only the salient-set check goes on."""
    import os
    import sys

    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
    import make_token_golden as mtg
    from oracle import dyllm_oracle as orc

    from dyllm_b200 import _lib, ops, runner
    from dyllm_b200.model import LLaDAForDLM, LLaDAShape

    fx = torch.load(os.path.join(os.path.dirname(__file__), "golden", "llada_tokens_small.pt"))
    c = mtg.CFG
    assert fx["cfg"] == c
    shape = LLaDAShape(hidden_size=c["hidden"], num_attention_heads=c["heads"], n_kv_heads=c["kv_heads"],
                       head_dim=c["head_dim"], mlp_hidden_size=c["inter"], num_hidden_layers=c["layers"],
                       vocab_size=c["vocab"], mask_token_id=mtg.MASK_ID, max_sequence_length=c["max_pos"],
                       rms_norm_eps=c["eps"], rope_theta=c["theta"])
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(cuda_device):
            model = LLaDAForDLM(shape, c["tau"])
    finally:
        torch.set_default_dtype(torch.float32)
    mtg.load_weights_into(model, {k: v.to(cuda_device) for k, v in mtg.token_model_weights().items()})
    model.eval()
    sr = runner.StepRunner(model, mtg.MASK_ID, block_length=c["block"], steps=c["steps"], num_full_steps=c["full_steps"],
                           refresh_period=4, use_graphs=False)
    sr.record_candidates = True
    prompts = mtg.token_prompts()
    seqs = sr.new_batch(prompts, c["gen"])
    seen = []
    real_select = ops.salient_select

    def recording_select(stats, threshold, *a, **k):
        sel = real_select(stats, threshold, *a, **k)
        seen.append((orc.cosine_values(stats.cpu()).float(), sel.idx[: int(sel.count.item())].cpu()))
        return sel

    ops.salient_select = recording_select
    forked_at = None
    failures = []
    steps_before_fork = rows_compared = tokens_compared = picks_compared = 0
    try:
        for step, rec in enumerate(fx["steps"]):
            seen.clear()
            picks = sr.step_picks(seqs, forced=rec["picks"])
            for layer, ((cos_got, idx_got), cos_ref) in enumerate(zip(seen, rec["layer_cosines"])):
                m_ref = cos_ref < c["tau"]
                m_got = torch.zeros_like(m_ref)
                m_got[idx_got] = True
                clear = (cos_ref - c["tau"]).abs() >= 2e-3
                if forked_at is None:
                    assert torch.equal(m_got[clear], m_ref[clear]), f"step {step + 1} layer {layer}: salient sets differ"
                    if not torch.equal(m_got, m_ref):
                        forked_at = step + 1
                        print(f"step {step + 1} layer {layer}: a decision inside the band went the other way "
                              f"(cosine error max {float((cos_got - cos_ref).abs().max()):.2e})")
            if forked_at is not None and forked_at <= step + 1:
                continue
            steps_before_fork += 1
            cand_pos, conf, tok = sr.last_candidates
            for b, (got, want, (sel_margin, _)) in enumerate(zip(picks, rec["picks"], rec["margins"])):
                mine = {p: (float(conf[b, i]), int(tok[b, i])) for i, p in enumerate(cand_pos[b]) if conf[b, i] >= 0}
                ref = {p: (cf, tk, mg) for p, cf, tk, mg in rec["candidates"][b]}
                assert set(mine) == set(ref), f"step {step + 1} sequence {b}: candidate rows differ"
                errs = []
                for p, (cf, tk, mg) in ref.items():
                    errs.append(abs(mine[p][0] - cf) / cf)
                    rows_compared += 1
                    if mg >= 0.5:
                        tokens_compared += 1
                        if mine[p][1] != tk:
                            failures.append(f"step {step + 1} sequence {b} position {p}: token {mine[p][1]} != {tk} "
                                            f"(reference lead {mg:.2f}, confidence {mine[p][0]:.3f} vs {cf:.3f})")
                print(f"step {step + 1} ({rec['kind']}) sequence {b}: confidence errors max {max(errs):.3f} "
                      f"mean {sum(errs) / len(errs):.3f}")
                if not (max(errs) <= 0.25 and sum(errs) / len(errs) <= 0.08):
                    failures.append(f"step {step + 1} ({rec['kind']}) sequence {b}: confidence errors max {max(errs):.3f} "
                                    f"mean {sum(errs) / len(errs):.3f}")
                if sel_margin >= 0.25:
                    picks_compared += 1
                    if got != want:
                        failures.append(f"step {step + 1} sequence {b}: {got} != {want}")
    finally:
        ops.salient_select = real_select
    print(f"steps compared before the runs forked: {steps_before_fork} (fork at step {forked_at}); candidate confidences "
          f"compared {rows_compared}, tokens {tokens_compared}, row choices {picks_compared}")
    assert not failures, "\n".join(failures)
    assert steps_before_fork >= 6 and rows_compared >= 100 and tokens_compared >= 30
    assert [s.token_ids[s.num_prompt_tokens:] for s in seqs] == fx["final_tokens"]
    assert _lib.load().dyllm_device_status() == 0
    # free-running generations (host-driven and device-resident) for the record
    sr.record_candidates = False
    total = c["batch"] * c["gen"]
    for device_state in (False, True):
        free = sr.generate(prompts, c["gen"], device_state=device_state)
        same = sum(a == b for row, ref in zip(free, fx["final_tokens"]) for a, b in zip(row, ref))
        print(f"free-running (device_state={device_state}): {same}/{total} final tokens equal the reference's")


def test_two_batch_geometries_on_one_model(cuda_device):
    """A second generation with another batch size and other lengths on the same model: the caches forget
    the first batch (sequence ids are reused) and captured graphs of the first geometry are dropped."""
    from dyllm_b200 import _lib, runner
    from dyllm_b200.model import LLaDAForDLM, LLaDAShape, init_weights_

    shape = LLaDAShape(hidden_size=256, num_attention_heads=2, n_kv_heads=2, head_dim=128, mlp_hidden_size=512,
                       num_hidden_layers=2, vocab_size=1024, mask_token_id=1000, max_sequence_length=256)
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(cuda_device):
            model = LLaDAForDLM(shape, 0.99)
    finally:
        torch.set_default_dtype(torch.float32)
    init_weights_(model, seed=5, std=0.05)
    model.eval()
    g = torch.Generator().manual_seed(1)
    small = torch.randint(0, 900, (2, 24), generator=g).tolist()
    large = torch.randint(0, 900, (5, 56), generator=g).tolist()

    def fresh():
        return runner.StepRunner(model, shape.mask_token_id, block_length=8, steps=16, num_full_steps=4, refresh_period=4,
                                 use_graphs=True)

    sr = fresh()
    want_small = sr.generate(small, 16)
    want_large = fresh().generate(large, 16)          # another runner of the same model, another geometry
    assert sr.generate(small, 16) == want_small       # the first runner notices that its graphs are stale
    sr3 = fresh()
    assert sr3.generate(small, 16) == want_small
    assert sr3.generate(small, 16) == want_small      # replay of the captured graphs
    assert sr3.generate(large, 16) == want_large      # longer sequences, more of them, same ids
    assert sr3.generate(small, 16) == want_small      # and back
    assert _lib.load().dyllm_device_status() == 0
