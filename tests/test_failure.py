"""Failure detection without faulting a GPU.

Host side (gloo ranks): a rank that raises is reported with its traceback; a rank that never joins a collective makes
the others fail by the process-group timeout instead of hanging; DDP refuses a step whose buckets did not all launch;
a torn checkpoint is never resumed from.  Device side: a collective kernel whose peer flag never arrives gives up
after its (short) wait limit, records a status word that the host reads, and leaves the context usable.
"""

import time

import pytest
import torch

from tests.dist_utils import run_distributed


def _one_rank_raises(rank, world):
    if rank == 1:
        raise ValueError("injected failure on rank 1")
    time.sleep(0.2)


def test_raising_rank_is_reported():
    with pytest.raises(AssertionError, match="injected failure on rank 1"):
        run_distributed(_one_rank_raises, 2, timeout_s=30)


def _missing_rank(rank, world, report_path):
    import json
    import os

    from torchure_b200.core.collective import all_reduce
    from torchure_b200.core.mesh import Mesh

    mesh = Mesh({"dp": world})
    if rank == 1:
        # leaves between steps: never joins the next collective, but stays alive until the survivor has reported, so
        # that only the process-group timeout (not a closed socket) can end the survivor's collective
        deadline = time.time() + 60
        while not os.path.exists(report_path) and time.time() < deadline:
            time.sleep(0.05)
        os._exit(0)  # no closing barrier: this rank takes part in no further collective
    t0 = time.time()
    raised = ""
    try:
        all_reduce(torch.ones(4), mesh, "dp", "sum")
    except Exception as e:  # the timeout of the process group
        raised = type(e).__name__
    with open(report_path + ".tmp", "w") as f:
        json.dump({"raised": raised, "seconds": time.time() - t0}, f)
    os.replace(report_path + ".tmp", report_path)
    os._exit(0)


def test_absent_rank_ends_collective_by_timeout(tmp_path):
    """A rank that silently stops joining collectives must not hang the others: the survivor's all_reduce raises
    within the process-group timeout (3 s here), and both ranks exit on their own."""
    import json

    report = str(tmp_path / "survivor.json")
    run_distributed(_missing_rank, 2, report, timeout_s=3, join_s=90)   # raises if a rank had to be terminated or crashed
    with open(report) as f:
        rec = json.load(f)
    assert rec["raised"], "the survivor's all_reduce returned although its peer never joined"
    assert rec["seconds"] < 9, f"the collective ended only after {rec['seconds']:.1f} s: not the 3 s timeout"


def test_torn_checkpoint_is_not_resumed(tmp_path):
    from torchure_b200.ckpt import Checkpointer

    ck = Checkpointer(str(tmp_path))
    ck.save_trainer({"step": 5}, 5)
    ck.mark_complete(5)
    ck.save_trainer({"step": 9}, 9)  # the writer died before the marker
    assert ck.latest() == 5 and ck.valid_step(9) is None


def _resume_faults(rank, world, home):
    import os

    os.environ["TORCHURE_B200_HOME"] = home
    from tests.tiny import parity_config
    from torchure_b200.train.trainer import Trainer

    first = Trainer(parity_config(2, steps=4, run_name="faults", accumulation=1, save_steps=2), rank, rank, world,
                    device="cpu")
    first.num_train_steps = 2
    first.train()
    # a relaunch on another mesh must refuse the checkpoint instead of loading tensors of the wrong shape
    other = parity_config(1, steps=4, run_name="faults", accumulation=2, resume="auto", mesh={"dp": 1, "tp": 2})
    with pytest.raises(AssertionError, match="mesh change"):
        Trainer(other, rank, rank, world, device="cpu")
    # a checkpoint that lost this rank's dataloader position must not silently restart the data from the beginning
    torch.distributed.barrier()
    if rank == 1:
        os.remove(os.path.join(home, "checkpoints", "faults", "2", "dataloader_dp1.pt"))
    torch.distributed.barrier()
    same = parity_config(2, steps=4, run_name="faults", accumulation=1, resume="auto")
    if rank == 1:
        with pytest.raises(FileNotFoundError):
            Trainer(same, rank, rank, world, device="cpu")
    else:
        assert Trainer(same, rank, rank, world, device="cpu").start_step == 2


def test_resume_refuses_another_mesh_and_a_missing_dataloader_file(tmp_path):
    run_distributed(_resume_faults, 2, str(tmp_path), timeout_s=120)


def test_config_errors_are_loud():
    from torchure_b200.config import ConfigError, validate_config
    from tests.tiny import parity_config

    cfg = parity_config(2)
    validate_config(cfg, 2)
    with pytest.raises(ConfigError):
        validate_config(cfg, 3)
    bad = parity_config(2)
    bad["data"]["global_batch_size"] = 6
    with pytest.raises(ConfigError):
        validate_config(bad, 2)
    bad = parity_config(2)
    del bad["mesh"]["dp"]
    bad["mesh"]["tp"] = 2
    with pytest.raises(ConfigError):
        validate_config(bad, 2)
    for mesh in ({"dp": 1, "ep": 2}, {"dp_shard": 1, "tp": 2}):      # nothing to select / not combinable
        with pytest.raises(ConfigError):
            validate_config(parity_config(1, mesh=mesh), 2)
    # context and pipeline parallelism: {"dp", "cp"} / {"dp", "pp"} in this order, chunks and stages that divide
    validate_config(parity_config(1, mesh={"dp": 1, "cp": 2}), 2)
    validate_config(parity_config(1, mesh={"dp": 1, "pp": 2}), 2)
    for mesh in ({"cp": 2, "dp": 1}, {"dp": 1, "tp": 1, "cp": 2}, {"pp": 2, "dp": 1}):
        with pytest.raises(ConfigError):
            validate_config(parity_config(1, mesh=mesh), 2)
    bad = parity_config(1, mesh={"dp": 1, "cp": 3})
    bad["data"]["seq_len"] = 256            # not a multiple of 2 x 3 chunks
    with pytest.raises(ConfigError):
        validate_config(bad, 3)
    bad = parity_config(1, mesh={"dp": 1, "cp": 4})     # two KV heads cannot be split four ways
    bad["cp"] = {"kind": "ulysses"}
    with pytest.raises(ConfigError):
        validate_config(bad, 4)
    bad = parity_config(1, mesh={"dp": 1, "pp": 8})     # four blocks
    with pytest.raises(ConfigError):
        validate_config(bad, 8)
    bad = parity_config(1, mesh={"dp": 1, "pp": 2})
    bad["pp"] = {"schedule": "zero-bubble"}
    with pytest.raises(ConfigError):
        validate_config(bad, 2)


def test_shipped_configs_validate():
    """Every file under configs/ (the reference-schema ones and the synthetic ones per strategy) passes validation for
    the world size its mesh spans."""
    import glob
    import json
    import math
    import os

    from torchure_b200.config import validate_config

    files = sorted(glob.glob(os.path.join(os.path.dirname(os.path.dirname(__file__)), "configs", "*.json")))
    assert len(files) >= 12
    for f in files:
        with open(f) as fh:
            cfg = json.load(fh)
        validate_config(cfg, math.prod(cfg["mesh"].values()))


@pytest.mark.gpu
def test_device_wait_expires_with_status_and_context_survives():
    """A barrier that expects a peer that does not exist: nothing ever sets the flag, the bounded wait runs out after
    50 ms, the kernel records the status word and returns; the next kernel on the same context works."""
    from torchure_b200 import ops

    ext = ops.ext()
    buf = torch.zeros(ext.COMM_FLAG_BYTES + ext.COMM_PARTIAL_BYTES, dtype=torch.uint8, device="cuda")
    word = ext.comm_error_word()
    word.zero_()
    t0 = time.time()
    ext.comm_barrier([buf.data_ptr()], 0, 0, 1, 50_000_000, 2)  # world 1, pretend there are 2 ranks, 50 ms limit
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    assert int(word[0].item()) == 5, "kErrPeerFlagWait must be recorded"
    word.zero_()
    x = torch.ones(1024, device="cuda")
    assert float((x * 2).sum().item()) == 2048.0  # the context is alive
    ext.comm_barrier([buf.data_ptr()], 0, 0, 1, 50_000_000, 1)  # a barrier with no missing peer passes
    torch.cuda.synchronize()
    assert int(word[0].item()) == 0
