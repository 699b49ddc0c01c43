"""world_size-2 gloo test of the calibration combine logic (no GPU): each rank holds half of the
images, statistics are combined with all-reduce(MAX) over packed (-min, max) and all-reduce(SUM)
over the int64 histograms; the result must equal the single-process statistics over all images."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

NAMES = ["a", "b", "zeros"]


def _activations(seed_base, n_images):
    out = []
    for i in range(n_images):
        rng = np.random.default_rng(seed_base + i)
        out.append({"a": rng.normal(0, 1 + i, (4, 8)).astype(np.float32),
                    "b": np.maximum(rng.normal(0, 2, (3, 5, 5)), 0).astype(np.float32),
                    "zeros": np.zeros((6,), np.float32)})
    return out


class _FakeModel:
    """Stands in for tpu_compiler_b200.module: no device, activations come from numpy."""
    _device = None
    op_info = [{"name": n, "dtype": "FP32"} for n in NAMES]

    def get_input_details(self):
        return ["data"]


def _make_calibrator(acts, d):
    from tpu_compiler_b200.calibration import ActivationCalibrator

    class CpuCal(ActivationCalibrator):
        def _local_min_max(self):
            st = torch.empty((len(self.names), 2), dtype=torch.float32)
            for t, n in enumerate(self.names):
                allv = np.concatenate([a[n].reshape(-1) for a in acts])
                st[t, 0], st[t, 1] = float(allv.min()), float(allv.max())
            return st, len(acts)

        def _local_histograms(self, stats, release=True):
            import oracle
            h = torch.zeros((len(self.names), self.bin_num), dtype=torch.int64)
            for t, n in enumerate(self.names):
                for a in acts:
                    h[t] += torch.from_numpy(oracle.histogram(a[n], float(stats[n][2]), self.bin_num))
            return h

        def find_threshold(self, hist, stats):
            return {n: float(hist[t].sum()) for t, n in enumerate(self.names)}

    return CpuCal(_FakeModel(), lambda: iter(()), 2048, input_name="data", dist=d)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    acts = _activations(100, 6)[rank::world]
    cal = _make_calibrator(acts, dist)
    stats = cal.find_min_max_abs()
    hist = cal.calc_histograms(stats)
    q.put((rank, {k: tuple(float(x) for x in v) for k, v in stats.items()}, hist.numpy(), cal.num_samples))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_statistics_equal_single_process():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    single = _make_calibrator(_activations(100, 6), None)
    s_stats = single.find_min_max_abs()
    s_hist = single.calc_histograms(s_stats).numpy()
    for rank, stats, hist, n in results:
        assert n == 6
        for k in NAMES:
            assert stats[k] == tuple(float(x) for x in s_stats[k]), (rank, k)
        assert np.array_equal(hist, s_hist)
    assert s_stats["zeros"] == (np.float32(-1e-5), np.float32(1e-5), np.float32(1e-5))


def _mismatch_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    from tpu_compiler_b200.calibration import join_ranks
    d = join_ranks("gloo", rank, world, timeout_s=30)
    cal = _make_calibrator(_activations(100, 2), d)
    if rank == 1:
        cal.names = cal.names[:-1]          # this rank loaded a module with one tensor less
    try:
        cal._check_ranks_agree()     # what the constructor runs; here after the lists were made to differ
        q.put((rank, "no error"))
    except RuntimeError as e:
        q.put((rank, str(e)))
    d.barrier()
    d.destroy_process_group()


def test_rank_mismatch_is_an_error_on_every_rank():
    """Host-side fault: two ranks that calibrate different tensor lists. Both must fail with the same plain message
    before any statistics are combined; neither may hang."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29950 + os.getpid() % 40
    procs = [ctx.Process(target=_mismatch_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert "ranks disagree" in results[0] and "ranks disagree" in results[1]
    assert "2..3" in results[0]


def _lonely_worker(port, q):
    import time
    from tpu_compiler_b200.calibration import join_ranks
    t0 = time.time()
    try:
        join_ranks("gloo", 0, 2, timeout_s=3, init_method="tcp://127.0.0.1:%d" % port)
        q.put(("joined", time.time() - t0))
    except RuntimeError as e:
        q.put((str(e), time.time() - t0))


def test_a_rank_that_never_joins_times_out_with_an_error():
    """Host-side fault: rank 1 of 2 never starts. Rank 0 gives up after the limit with an error; no hang."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_lonely_worker, args=(29990 + os.getpid() % 9, q))
    p.start()
    msg, seconds = q.get(timeout=90)
    p.join(timeout=30)
    assert p.exitcode == 0
    assert "not all 2 ranks joined within 3 s" in msg and seconds < 60
