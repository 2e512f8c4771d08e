"""The native-torch conformance model (tests/autograd_reference.py) checked against itself on CPU:
with a row-local attention, a context-parallel group must produce what one device produces on the
whole sequence -- the routes of the model are then the Ulysses routes, not just self-consistent."""
import torch

from tests.autograd_reference import reference_world


def test_context_parallel_model_equals_single_device_model():
    torch.manual_seed(7)
    cp, seq, hidden, q_heads, kv_heads, d = 4, 6, 24, 8, 4, 4
    xs = [torch.randn(seq, hidden, dtype=torch.float64) for _ in range(cp)]
    dys = [torch.randn(seq, hidden, dtype=torch.float64) for _ in range(cp)]
    w_qkv = torch.randn((q_heads + 2 * kv_heads) * d, hidden, dtype=torch.float64)
    w_o = torch.randn(hidden, q_heads * d, dtype=torch.float64)
    many = reference_world(xs, w_qkv, w_o, dys, cp=cp, seq_local=seq, q_heads=q_heads, kv_heads=kv_heads, head_dim=d)
    one = reference_world([torch.cat(xs)], w_qkv, w_o, [torch.cat(dys)], cp=1, seq_local=seq * cp, q_heads=q_heads,
                          kv_heads=kv_heads, head_dim=d)[0]
    ql, kvl = q_heads // cp * d, kv_heads // cp * d
    for r in range(cp):
        rows = slice(r * seq, (r + 1) * seq)
        torch.testing.assert_close(many[r]["y"], one["y"][rows])
        torch.testing.assert_close(many[r]["dx"], one["dx"][rows])
        torch.testing.assert_close(many[r]["q"], one["q"][:, r * ql:(r + 1) * ql])
        torch.testing.assert_close(many[r]["k"], one["k"][:, r * kvl:(r + 1) * kvl])
        torch.testing.assert_close(many[r]["v"], one["v"][:, r * kvl:(r + 1) * kvl])
    # weight gradients are per rank (no cross-rank reduction in the operators): their sum is the whole
    torch.testing.assert_close(sum(m["dw_qkv"] for m in many), one["dw_qkv"])
    torch.testing.assert_close(sum(m["dw_o"] for m in many), one["dw_o"])
