"""Case table and input helpers shared by the golden generator and the tests (no reference import)."""
from oracle import moe_oracle as O

# name -> (T, H, E, I, k, seed, bias_std, cap)   cap: route only to experts < cap (empty experts)
CASES = {
    "cfg1": (512, 256, 8, 512, 2, 0, 0.01, None),          # benchmark config 1
    "situ_small": (512, 128, 6, 96, 2, 7, 0.0, None),      # parity_situ.py:12 shape
    "empty_experts": (512, 128, 6, 96, 2, 7, 0.0, 4),      # parity_situ.py:93 (experts 4,5 empty)
    "grouped_k4": (1024, 128, 16, 64, 4, 3, 0.01, None),   # top-4, more experts
}


def sub(t):
    """Sub-sample of a large (E, rows, cols) weight gradient kept in the fixture."""
    return t[:, ::8, ::8].contiguous()


def routing_for(inp, E, k, cap):
    """Routing fed to the reference's moe_eager when the fixture was made."""
    logits = inp["x"] @ inp["gate_weight"].t()
    if cap is not None:
        logits = logits.clone()
        logits[:, cap:] = -1e4                 # sigmoid -> 0: never picked while cap >= k
    idx, w, counts = O.router_epilogue_fwd(logits, inp["bias"], k)
    return idx, w
