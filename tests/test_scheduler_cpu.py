"""CPU tests of the view scheduler's host logic: sharding arithmetic, the broadcast + shard
protocol over a world_size-2 gloo group, and the ViewScheduler class itself driven through an
injected host-only session (scene broadcast, view sharding, and a rank whose render call fails:
its undone views are re-issued to the surviving rank). No GPU, no kernels; the failure is an
exception raised on the host, between views."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from renderformer_cuda_b200 import session


def test_shard_views_partitions_every_view_once():
    for n, world in [(64, 8), (64, 3), (5, 8), (0, 2), (7, 1)]:
        seen = []
        for r in range(world):
            mine = session.shard_views(n, r, world)
            assert all(v % world == r for v in mine)
            seen += mine
        assert sorted(seen) == list(range(n))
        sizes = [len(session.shard_views(n, r, world)) for r in range(world)]
        assert max(sizes) - min(sizes) <= 1


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # the scene state travels as one byte blob from rank 0; every rank ends with identical bytes
    state = torch.arange(4096, dtype=torch.uint8) if rank == 0 else torch.zeros(4096, dtype=torch.uint8)
    dist.broadcast(state, src=0)
    mine = session.shard_views(11, rank, world)
    # a stand-in "render": each rank fills its own views, then the host gathers them
    frames = torch.zeros(11, 4)
    for v in mine:
        frames[v] = float(v) + state[:4].float()
    dist.all_reduce(frames)
    ret[rank] = (int(state.sum()), mine, frames.tolist())
    dist.destroy_process_group()


def test_broadcast_and_shard_protocol_gloo_world2():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret[0][0] == ret[1][0] == int(torch.arange(4096, dtype=torch.uint8).sum())
    assert ret[0][1] == [0, 2, 4, 6, 8, 10] and ret[1][1] == [1, 3, 5, 7, 9]
    want = [[float(v) + i for i in range(4)] for v in range(11)]
    assert ret[0][2] == want and ret[1][2] == want


class FakeSession:
    """Host-only stand-in for RenderSession: the 'frame' of a view is its fov plus one byte of the scene state."""

    def __init__(self, scene_state, fail_after=None):
        self.scene_state = scene_state if scene_state is not None else torch.zeros(64, dtype=torch.uint8)
        self.fail_after, self.count, self.last_fov, self.finalized = fail_after, 0, None, False

    def encode_scene(self, tri, vn, tex):
        self.scene_state.copy_(torch.arange(64, dtype=torch.uint8) + 3)

    def finalize(self):
        self.finalized = True

    def render_frame_raw(self, c2w_ptr, fov):
        assert self.finalized
        if self.fail_after is not None and self.count >= self.fail_after:
            raise session.RfkLayersError("injected failure of this rank's device")
        self.count += 1
        self.last_fov = fov

    def download_async(self, host):
        host.fill_(self.last_fov + float(self.scene_state[1]))

    def drain(self):
        pass

    def close(self):
        pass


def _sched_worker(rank, world, port, ret, fail_rank, streams):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    V = 11
    factory = lambda st: FakeSession(st, fail_after=2 if rank == fail_rank else None)
    sched = session.ViewScheduler(None, 0, session_factory=factory, streams_per_gpu=streams)
    sched.load_scene("tri", "vn", "tex")              # rank 0 encodes, the state travels, every session finalizes
    state_ok = bool((sched.session.scene_state == torch.arange(64, dtype=torch.uint8) + 3).all())
    shared = all(s.scene_state is sched.session.scene_state for s in sched.sessions)
    out = torch.zeros(V, 4)
    try:
        done = sched.render(torch.zeros(V, 4, 4), torch.arange(V, dtype=torch.float32), out)
        err = None
    except session.SchedulerError as e:
        done, err = [], str(e)
    rows_ok = all(float(out[i, 0]) == float(v) + 4.0 for i, v in enumerate(done))
    ret[rank] = (state_ok and shared, done, rows_ok, sched.failed, err)
    dist.barrier()
    dist.destroy_process_group()


def _run_sched(fail_rank, streams=1):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_sched_worker, args=(2, port, ret, fail_rank, streams), nprocs=2, join=True)
    return ret


def test_view_scheduler_class_world2_no_failure():
    ret = _run_sched(fail_rank=-1, streams=2)
    assert ret[0][0] and ret[1][0]
    assert ret[0][1] == [0, 2, 4, 6, 8, 10] and ret[1][1] == [1, 3, 5, 7, 9]
    assert ret[0][2] and ret[1][2] and not ret[0][3] and not ret[1][3]


def test_view_scheduler_reissues_views_of_a_failed_rank():
    ret = _run_sched(fail_rank=1)
    assert ret[0][0] and ret[1][0]
    # rank 1 rendered its first two views, then its session raised: views 5, 7, 9 go to the survivor
    assert ret[1][1] == [1, 3] and ret[1][3] is True and ret[1][4] is None
    assert ret[0][1] == [0, 2, 4, 6, 8, 10, 5, 7, 9] and ret[0][3] is False
    assert ret[0][2] and ret[1][2]                    # every downloaded row belongs to the view listed for it
    assert sorted(ret[0][1] + ret[1][1]) == list(range(11))


def test_view_scheduler_single_rank_failure_raises():
    sched = session.ViewScheduler(None, 0, session_factory=lambda st: FakeSession(st, fail_after=1))
    sched.load_scene("tri", "vn", "tex")
    try:
        sched.render(torch.zeros(3, 4, 4), torch.arange(3, dtype=torch.float32))
        raised = False
    except session.SchedulerError as e:
        raised = "[1, 2]" in str(e)
    assert raised


class FakeBatchedSession(FakeSession):
    """Stand-in for a session whose frame holds several views: a frame's rows are its views' fovs plus one scene byte."""

    def __init__(self, scene_state, views, fail_after=None):
        super().__init__(scene_state, fail_after)
        self.views, self.frames = views, []

    def render_frames_raw(self, cams_ptr, fovs_ptr):
        import ctypes
        assert self.finalized
        if self.fail_after is not None and self.count >= self.fail_after:
            raise session.RfkLayersError("injected failure of this rank's device")
        self.count += 1
        self.last_fovs = list((ctypes.c_float * self.views).from_address(fovs_ptr))
        cams = list((ctypes.c_float * (16 * self.views)).from_address(cams_ptr))
        self.frames.append((self.last_fovs, cams[::16]))          # element [0,0] of each camera carries its view id

    def download_async(self, host):
        assert host.shape[0] == self.views
        for i, f in enumerate(self.last_fovs):
            host[i].fill_(f + float(self.scene_state[1]))


def _batched(n_views, per_frame, streams=1, fail_after=None):
    made = []

    def factory(st):
        made.append(FakeBatchedSession(st, per_frame, fail_after))
        return made[-1]
    sched = session.ViewScheduler(None, 0, session_factory=factory, streams_per_gpu=streams, views_per_frame=per_frame)
    sched.load_scene("tri", "vn", "tex")
    c2ws = torch.zeros(n_views, 4, 4)
    c2ws[:, 0, 0] = torch.arange(n_views, dtype=torch.float32)
    return sched, made, c2ws, torch.arange(n_views, dtype=torch.float32)


def test_view_scheduler_cuts_views_into_frames_and_pads_the_last_one():
    for n_views, per_frame, streams in [(8, 4, 1), (11, 4, 2), (3, 4, 1), (5, 2, 3)]:
        sched, made, c2ws, fovs = _batched(n_views, per_frame, streams)
        out = torch.full((n_views, 4), -1.0)
        done = sched.render(c2ws, fovs, out)
        assert done == list(range(n_views))
        assert torch.equal(out, (fovs + 4.0)[:, None].expand(n_views, 4))    # padded views never reach `out`
        frames = [f for s in made for f in s.frames]
        assert len(frames) == -(-n_views // per_frame)
        assert [len(s.frames) for s in made] == [len(range(i, len(frames), streams)) for i in range(streams)]
        for fv, cam_ids in frames:
            assert fv == cam_ids                      # every camera travelled with its own fov
        tail = max(frames, key=lambda f: f[0][0])[0]
        assert tail[-1] == float(n_views - 1) and all(v == tail[-1] for v in tail[(n_views - 1) % per_frame:])


def test_view_scheduler_batched_single_rank_failure_raises():
    sched, made, c2ws, fovs = _batched(9, 4, fail_after=1)
    try:
        sched.render(c2ws, fovs, torch.zeros(9, 4))
        raised = False
    except session.SchedulerError:
        raised = True
    assert raised and sched.failed and made[0].count == 1
