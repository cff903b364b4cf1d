"""Counter-based uniform numbers for sampling, keyed by (seed, request, token
index): a request draws the same numbers however it was batched, cut into
portions, or preempted and recomputed.  (The reference shares one mt19937 over
the batch, src/models/gpt_model.cpp:128-129, so its draws depend on the batch.)

Three rounds of the splitmix64 finaliser; the top 24 bits give a float32-exact
number in [0, 1).
"""
_MASK = (1 << 64) - 1


def _mix(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform(seed: int, request: int, index: int) -> float:
    z = _mix(seed & _MASK)
    z = _mix(z ^ (request & _MASK))
    z = _mix(z ^ (index & _MASK))
    return (z >> 40) / float(1 << 24)
