"""Protocol models of the single-launch backward kernels (see tests/protocol_models.py): random
shapes, random durations, any number of resident blocks per GPU."""
import random

import pytest

from tests import protocol_models as pm


def _shard_case(seed):
    rnd = random.Random(seed)
    R, P, U = rnd.randint(2, 4), rnd.randint(1, 6), rnd.randint(2, 12)
    E, C = rnd.randint(1, 3), rnd.randint(1, 3)
    conv_off = rnd.randint(0, U)
    ns = rnd.randint(2, 4)
    return dict(R=R, P=P, U=U, E=E, C=C, exch_off=rnd.randint(0, conv_off), conv_off=conv_off, slots=rnd.randint(1, 12), seed=seed,
                ns=ns, lag=rnd.randint(1, ns - 1))


@pytest.mark.parametrize("in_place", [False, True])
def test_sharded_exchange_has_no_deadlock_and_no_buffer_hazard(in_place):
    for seed in range(150):
        pm.run_sharded(in_place=in_place, **_shard_case(seed))


def test_flags_must_be_published_in_slot_order():
    """Without the rule that a rank publishes its flags strictly in slot order, a late block of an
    early slot lets a peer overwrite a buffer that is still being read: the model finds it."""
    hazards = 0
    for seed in range(150):
        try:
            pm.run_sharded(in_place=True, ordered=False, **_shard_case(seed))
        except pm.Hazard:
            hazards += 1
    assert hazards > 0


def test_pipelined_backward_never_waits_for_a_later_block():
    for seed in range(300):
        rnd = random.Random(seed)
        U = rnd.randint(1, 30)
        ns = rnd.randint(2, 4)
        pm.run_pipelined(P=rnd.randint(1, 8), U=U, C=rnd.randint(1, 6), conv_off=rnd.randint(0, U), slots=rnd.randint(1, 20),
                         seed=seed, ns=ns, lag=rnd.randint(1, ns - 1))


def test_small_allreduce_needs_only_two_cells_per_sender():
    for seed in range(200):
        rnd = random.Random(seed)
        pm.run_small_allreduce(R=rnd.randint(2, 8), calls=rnd.randint(1, 12), seed=seed)
