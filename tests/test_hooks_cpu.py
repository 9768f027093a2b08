"""Model-side hooks (sageattention_b200/hooks.py) on CPU: which attention function gets called when.  No kernel
runs here; the functions are stand-ins that record their calls."""
import torch
import torch.nn.functional as F

from sageattention_b200 import hooks


def _recorder(tag, log):
    def fn(q, k, v, *a, **kw):
        log.append((tag, kw))
        return q
    return fn


def test_sdpa_adapter_routes_unsupported_cases_to_the_precise_function():
    log = []
    sdpa = hooks.as_sdpa(attn_fn=_recorder("fp4", log), precise_fn=_recorder("precise", log))
    q = torch.zeros(1, 2, 8, 64, dtype=torch.bfloat16)
    sdpa(q, q, q)                                           # CPU tensor: not for the FP4 operator
    sdpa(q, q, q, attn_mask=torch.zeros(8, 8, dtype=torch.bool))
    assert [t for t, _ in log] == ["precise", "precise"]
    assert log[1][1]["attn_mask"] is not None


def test_patched_sdpa_is_undone_on_exit():
    original = F.scaled_dot_product_attention
    log = []
    with hooks.patched_sdpa(_recorder("patched", log)):
        q = torch.zeros(1, 1, 4, 8)
        F.scaled_dot_product_attention(q, q, q)
    assert F.scaled_dot_product_attention is original and [t for t, _ in log] == ["patched"]


def test_hybrid_schedule_uses_the_precise_function_at_the_first_and_last_steps():
    log = []
    h = hooks.TimestepHybridAttention(6, fast_fn=_recorder("fast", log), precise_fn=_recorder("precise", log),
                                      first=1, last=2)
    q = torch.zeros(1, 1, 4, 8)
    for step in range(6):
        h.set_step(step)
        h(q, q, q, is_causal=False)
    assert [t for t, _ in log] == ["precise", "fast", "fast", "fast", "precise", "precise"]
    assert h.calls == {"fast": 3, "precise": 3}


def test_set_attn_func_reaches_every_processor():
    class Proc:
        def __init__(self):
            self.attn_func = None

    class Attn(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.processor = Proc()

    model = torch.nn.Sequential(Attn(), torch.nn.Linear(2, 2), Attn())
    fn = lambda *a, **k: None
    assert hooks.set_attn_func(model, fn) == 2
    assert all(m.processor.attn_func is fn for m in model if isinstance(m, Attn))
