"""The peer-memory flag protocols of the NVSwitch kernels under the CPU simulator: the forms the kernels use are free of
unordered accesses and stale reads under random schedules at 2, 4 and 8 ranks; for each, a form without the ordering the
protocol relies on is reported."""

import pytest

from pear_b200.utils.protocol_sim import PROTOCOLS, ProtocolError, Sim, check, device_barrier, main, record_exchange


@pytest.mark.parametrize("name", sorted(PROTOCOLS))
@pytest.mark.parametrize("world", [2, 4, 8])
def test_protocol_is_ordered_and_its_broken_form_is_reported(name, world):
    prog, good, broken = PROTOCOLS[name]
    check(prog, world, schedules=40, **good)
    with pytest.raises(ProtocolError):
        check(prog, world, schedules=40, **broken)


def test_an_even_number_of_exchanges_per_step_meets_the_same_buffer_and_stays_ordered():
    for kinds in (2, 3, 4):
        check(record_exchange, 4, schedules=40, kinds=kinds, buffers=2)
    check(record_exchange, 4, schedules=40, kinds=2, buffers=1)  # ordered by the other exchange's barrier, even with one buffer


def test_detector_reports_each_kind_of_error():
    def unordered_read(rank, world):
        if rank == 0:
            yield ("write", "x", 1)
        else:
            yield ("read", "x", 1)

    def stale(rank, world):
        if rank == 0:
            yield ("write", "x", 1)
            yield ("signal", 1, 0, 1)
            yield ("wait", 0, 1, 1)
        else:
            yield ("wait", 0, 0, 1)
            yield ("read", "x", 2)
            yield ("signal", 0, 0, 1)

    def stuck(rank, world):
        yield ("wait", 0, 1 - rank, 1)

    def backwards(rank, world):
        yield ("signal", 1 - rank, 0, 2)
        yield ("signal", 1 - rank, 0, 1)

    for prog, msg in ((unordered_read, "not ordered before|before anything wrote"), (stale, "expected 2"), (stuck, "deadlock"), (backwards, "backwards")):
        with pytest.raises(ProtocolError, match=msg):
            check(prog, 2, schedules=20)
    # release / acquire is transitive: 0 -> 1 -> 2 orders rank 2's read after rank 0's write
    def chain(rank, world):
        if rank == 0:
            yield ("write", "x", 1)
            yield ("signal", 1, 0, 1)
        elif rank == 1:
            yield ("wait", 0, 0, 1)
            yield ("signal", 2, 0, 1)
        else:
            yield ("wait", 0, 1, 1)
            yield ("read", "x", 1)
    check(chain, 3, schedules=20)
    sim = Sim(2, 0)
    sim.run([iter(device_barrier(r, 2, 0, 1)) for r in range(2)])
    assert len(sim.trace) == 8


def test_command_line_reports_every_protocol(capsys):
    assert main(["--world", "2", "--schedules", "10"]) == 0
    out = capsys.readouterr().out
    assert all(name in out for name in PROTOCOLS) and "NOT reported" not in out and "FAILED" not in out
