"""The direct expert-parallel exchange has no back-pressure flag: a rank stores rows into a peer's slab for exchange e + 1
without asking whether the peer is done with exchange e, and an owner overwrites its per-route results for e + 1 while origins
read them over NVLink for e. This host-only model checks, under random skew between the ranks, that the order the protocol
does enforce (dispatch flag -> experts -> "results ready" flag -> combine, per rank in stream order) already makes both safe,
and that a flag word never runs ahead of the exchange number a waiting rank compares it with (the device waits for equality).

Per rank and exchange e the device stream runs, in order (forja_b200/csrc/fj_moe.cu, the direct branch of the step):
  A  ep_push_dispatch_kernel: stores into slab [dst][rank] of every dst, then dispatch-flag[dst][rank] = e
  B  ep_wait_kernel:          until dispatch-flag[rank][src] == e for every src
  C  expert kernels:          read slab [rank][*], write results[rank][*]
  D  ep_wait_kernel (signal): ready-flag[dst][rank] = e for every dst, then
  E                           until ready-flag[rank][owner] == e for every owner
  F  ep_pull_combine_kernel:  reads results[owner][rank] of every owner
"""
import random


def simulate(world, exchanges, rng):
    clock = [0.0] * world
    stage = [("A", 1)] * world                      # next operation of every rank: (name, exchange)
    dispatch_flag = [[(0, 0.0)] * world for _ in range(world)]   # [dst][src] = (value, time it was set)
    ready_flag = [[(0, 0.0)] * world for _ in range(world)]      # [dst][owner]
    slab_read_end = [[0.0] * world for _ in range(world)]        # [reader dst][src]: when dst finished reading src's slab
    slab_read_of = [[0] * world for _ in range(world)]           # ... for which exchange
    results_read_end = [[0.0] * world for _ in range(world)]     # [owner][origin]: when origin finished reading owner's results
    results_read_of = [[0] * world for _ in range(world)]
    done = [False] * world

    def jitter():
        return rng.choice([0.0, 0.1, 1.0, 5.0]) * rng.random()

    while not all(done):
        progressed = False
        for r in sorted(range(world), key=lambda i: clock[i]):
            if done[r]:
                continue
            op, e = stage[r]
            if op == "A":
                clock[r] += jitter()
                for dst in range(world):
                    # the store into dst's slab must not land while dst still reads the previous exchange from it
                    assert slab_read_of[dst][r] == e - 1, f"rank {r} dispatches {e} while rank {dst} has read only {slab_read_of[dst][r]}"
                    assert clock[r] >= slab_read_end[dst][r], f"rank {r} overwrites its slab at rank {dst} during exchange {e - 1}'s expert work"
                    assert dispatch_flag[dst][r][0] == e - 1
                    dispatch_flag[dst][r] = (e, clock[r])
                stage[r] = ("B", e)
            elif op == "B":
                if any(dispatch_flag[r][s][0] < e for s in range(world)):
                    continue                                     # blocked: some source has not dispatched yet
                assert all(dispatch_flag[r][s][0] == e for s in range(world)), "a dispatch flag ran ahead of the exchange waited for"
                clock[r] = max([clock[r]] + [dispatch_flag[r][s][1] for s in range(world)])
                stage[r] = ("C", e)
            elif op == "C":
                for origin in range(world):
                    # writing this exchange's results must not start while an origin still reads the previous ones
                    assert results_read_of[r][origin] == e - 1
                    assert clock[r] >= results_read_end[r][origin], f"rank {r} overwrites results that rank {origin} is still combining"
                clock[r] += 1.0 + jitter()
                for s in range(world):
                    slab_read_end[r][s], slab_read_of[r][s] = clock[r], e
                stage[r] = ("D", e)
            elif op == "D":
                for dst in range(world):
                    assert ready_flag[dst][r][0] == e - 1
                    ready_flag[dst][r] = (e, clock[r])
                stage[r] = ("E", e)
            elif op == "E":
                if any(ready_flag[r][o][0] < e for o in range(world)):
                    continue
                assert all(ready_flag[r][o][0] == e for o in range(world)), "a ready flag ran ahead of the exchange waited for"
                clock[r] = max([clock[r]] + [ready_flag[r][o][1] for o in range(world)])
                stage[r] = ("F", e)
            else:
                clock[r] += 0.5 + jitter()
                for owner in range(world):
                    results_read_end[owner][r], results_read_of[owner][r] = clock[r], e
                if e == exchanges:
                    done[r] = True
                else:
                    clock[r] += 2.0 * jitter()                   # attention and router of the next layer
                    stage[r] = ("A", e + 1)
            progressed = True
            break                                                # always advance the rank that is furthest behind
        assert progressed, "deadlock: every unfinished rank waits for a flag"
    return max(clock)


def test_slabs_and_results_are_never_overwritten_while_in_use_under_random_skew():
    for seed in range(40):
        rng = random.Random(seed)
        world = rng.choice([2, 3, 4, 8])
        assert simulate(world, exchanges=rng.choice([1, 3, 12]), rng=rng) > 0.0
