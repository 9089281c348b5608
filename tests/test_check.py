"""compatibility() on machines this one is not: every reason it says ok, untested or cannot run (the reference's
tests/test_check.py, re-targeted to compute capability 10.0)."""

from unicaattention_b200.check import OK, UNSUPPORTED, UNTESTED, compatibility

TESTED = {"platform": "linux", "torch": "2.11.0+cu128", "torch_cuda": "12.8", "gpu": "NVIDIA B200",
          "capability": (10, 0), "driver": 13000}


def judge(**changes):
    return compatibility(TESTED | changes)


def test_the_tested_machine_is_ok():
    assert judge() == (OK, ())
    assert judge(driver=13050).status == OK  # a newer driver runs older machine code


def test_untested_but_runs():
    for changes in ({"gpu": "NVIDIA GB200"}, {"driver": 12090}, {"torch": "2.15.0+cu132"}, {"platform": "win32"}):
        status = judge(**changes)
        assert status.status == UNTESTED and len(status.reasons) == 1, changes
    assert len(judge(platform="freebsd", gpu="NVIDIA B100").reasons) == 2


def test_cannot_run():
    for changes in ({"capability": (12, 0), "gpu": "NVIDIA GeForce RTX 5080"}, {"capability": (10, 3)}, {"capability": (9, 0)},
                    {"driver": 12040}, {"driver": None}, {"torch_cuda": None, "capability": None, "gpu": None},
                    {"capability": None, "gpu": None}):
        status = judge(**changes)
        assert status.status == UNSUPPORTED and status.reasons, changes
    # what cannot run is all that is said, not what is merely untested besides
    assert judge(capability=(8, 9), platform="freebsd").reasons == judge(capability=(8, 9)).reasons
    assert "cannot run" in str(judge(driver=None))
