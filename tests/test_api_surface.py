"""The names a user script of the reference imports exist here under ``necklace_b200`` with the
same spelling (reference: necklace/__init__.py, necklace/trainer/*.py, necklace/cuda/ncclgrp.py,
necklace/frmwrk/pytorch/mpnn/__init__.py:8-27, examples/*), and the log-channel numbers that
scripts pass to ``ilog.il_add`` are the reference's."""
import importlib

import pytest

SURFACE = {
    "": ["init", "init_mp", "init_nb"],
    "pympi.api": ["MpiWrp", "rank_size_from_env"],
    "utils.argutils": ["attach_nk_args_parser", "args_remake"],
    "utils.hookbase": ["NklcHookBase"],
    "utils.wrpbase": ["NklcWrapperBase"],
    "utils.tmrit": ["TimerItLogger"],
    "rpc.ilog": ["il_add", "il_del", "debug"],
    "rpc.svctmp": ["TmplServer", "TmplService", "TmplClient"],
    "cuda.ncclgrp": ["init_nccl_groups_map", "get_nccl_groups_map_cfg_dict",
                     "get_nccl_groups_map_grp_dict", "get_nccl_group_main_grp_list",
                     "get_nccl_group_dp", "get_nccl_group_mp", "get_nccl_group_pp",
                     "get_nccl_group_zr", "get_nccl_group_dp_or_main", "get_nccl_group_mp_or_main",
                     "get_nccl_group_pp_or_main", "get_nccl_group_zr_or_main", "get_rank",
                     "get_world_size", "NcclProcessGroup"],
    "cuda.ncclfns": ["all_gather", "all_reduce", "broadcast", "reduce", "pg_all_gather",
                     "pg_all_reduce", "pg_broadcast", "pg_reduce"], "cuda.ncclwrp": ["PYNCCL_DTYPE_MAP"], "cuda.quantize": ["CMP_RATIO", "cu_fn_matrix_quantize_e", "cu_fn_matrix_dequantize_e",
                      "cu_knl_matrix_quantize_e", "cu_knl_matrix_dequantize_e"],
    "cuda.nbutils": ["cuda_select_device", "cuda_current_context", "cuda_stream", "cuda_to_device",
                     "cuda_devarr_c_void_p"],
    "cuda.ncclutils": ["tensor_data_ptr", "tensor_size", "tensor_dtype", "nccl_all_reduce",
                       "nccl_all_gather", "nccl_reduce", "nccl_bcast", "nccl_reduce_scatter",
                       "seg_cb_nccl_ar", "nccl_out_all_gather"],
    "cuda.ncclpgs": ["NcclProcessGroup", "init_nccl_groups_map", "get_nccl_group_dp",
                     "get_nccl_group_mp", "get_nccl_group_dp_or_main", "get_nccl_group_mp_or_main",
                     "get_nccl_groups_map_cfg_dict", "get_nccl_groups_map_grp_dict", "get_rank",
                     "get_world_size", "ensure_divisibility", "divide", "build_pg_cfg"],
    "trainer.tndsnc": ["SVCScheduler", "SVCWorker"],
    "trainer.tndsms": ["SVCScheduler", "SVCWorker"],
    "trainer.tndsmp": ["MPSVCScheduler", "MPSVCWorker", "MPSVRScheduler", "MPSVRWorker"],
    "trainer.tndspp": ["MPSVCScheduler", "MPSVCWorker", "MPSVRScheduler", "MPSVRWorker"],
    "trainer.tndszr": ["MPSVCScheduler", "MPSVCWorker", "MPSVRScheduler", "MPSVRWorker"],
    "trainer.tndszd": ["MPSVCScheduler", "MPSVCWorker", "MPSVRScheduler", "MPSVRWorker"],
    "trainer.tnoppt": ["TrainerOPPytorch"],
    "trainer.mpoppt": ["TrainerMPOPPytorch"], "trainer.ppoppt": ["TrainerMPOPPytorch"],
    "trainer.zroppt": ["TrainerMPOPPytorch"], "trainer.zroppf": ["TrainerMPOPPytorch"],
    "trainer.zroppd": ["TrainerMPOPPytorch"], "trainer.tnmode": [],
    "frmwrk.pytorch.mpnn": [
        "destroy_model_parallel", "get_data_parallel_group", "get_data_parallel_rank",
        "get_data_parallel_world_size", "get_model_parallel_group", "get_model_parallel_rank",
        "get_model_parallel_src_rank", "get_model_parallel_world_size",
        "initialize_model_parallel", "model_parallel_is_initialized", "ColumnParallelLinear",
        "ParallelEmbedding", "RowParallelLinear", "VocabParallelEmbedding",
        "copy_to_model_parallel_region", "gather_from_model_parallel_region",
        "reduce_from_model_parallel_region", "scatter_to_model_parallel_region",
        "vocab_parallel_cross_entropy", "broadcast_data", "clip_grad_norm", "checkpoint",
        "get_cuda_rng_tracker", "model_parallel_cuda_manual_seed",
        "partition_activations_in_checkpoint"],
    "frmwrk.pytorch.mpnn.checkpointing": ["checkpoint", "get_cuda_rng_tracker",
                                          "model_parallel_cuda_manual_seed"],
    "frmwrk.pytorch.mpnn.samplers": [], "frmwrk.pytorch.mpnn.utils": [],
    "frmwrk.pytorch.ptutils": ["prnt_md"],
    "frmwrk.pytorch.dataldr": ["get_dist_dataloader"],
    "frmwrk.pytorch.callback": ["save_checkpoint"],
    "data.dtdummy": ["DtstDummy", "DtldDummy"],
    "data.dtqpto": ["DataLoaderSharedMemory"], "data.dtqptp": ["DataLoaderSharedMemory"],
    "data.dtmptp": ["DataLoaderSharedMemory"], "data.dtmptv": ["DataLoaderSharedMemory"],
    "data.sampler": [], "data.batchify": [], "data.shmem": [], "data.dtmem": ["DataLoaderSharedMemory", "DataLoaderShmForModule"], "data.dtshm": [],
    "data.dtshmp": [], "data.shmpt": [], "data.dtdist": [], "data.dtset": [], "data.dtwrp": [],
    "data.dtldngn": [], "data.shmmx": ["SharedMemArray"], "data.dtmmx": ["DataLoaderSharedMemory"],
    "data.dtmmxp": ["DataLoaderSharedMemory"], "data.dtexchg": ["DataExchanger"],
    "data.ptdlspn": [], "frmwrk.mxnet": [], "trainer.tnopmx": ["TrainerOPGluon"],
    "frmwrk.pytorch.ptmpi": ["params_do_mpi_allreduce", "opt_grads_do_mpi_allreduce",
                             "init_params_recvs", "init_opt_grads_recvs", "nccl_nc_allreduce",
                             "nccl_pg_allreduce", "nccl_pg_broadcast", "nccl_pg_reduce",
                             "opt_grads_do_nccl_allreduce", "opt_one_grads_do_nccl_allreduce",
                             "nccl_allreduce_by_buckets"],
    "frmwrk.pytorch.dtwrp": ["DataLoaderWrp", "DataLoaderIterWrp"],
    "frmwrk.pytorch.ptacts": [],
}

CHANNELS = {
    "tndsmp": {"ILOG_I_MP_SVR_WKR": 600001, "ILOG_I_MP_SVC_WKR": 600002,
               "ILOG_I_MP_SVR_SCH": 600003, "ILOG_I_MP_SVC_SCH": 600004},
    "tndspp": {"ILOG_I_MP_SVR_WKR": 600011, "ILOG_I_MP_SVR_WKR_PRT": 600015,
               "ILOG_I_MP_SVC_WKR": 600012, "ILOG_I_MP_SVC_WKR_PRT": 600016,
               "ILOG_I_MP_SVR_SCH": 600021, "ILOG_I_MP_SVR_SCH_PRT": 600025,
               "ILOG_I_MP_SVC_SCH": 600022, "ILOG_I_MP_SVC_SCH_PRT": 600026},
    "tndszr": {"ILOG_I_MP_SVR_WKR": 600001, "ILOG_I_ZR_SVR_WKR": 800001,
               "ILOG_I_ZR_SVC_WKR": 800002, "ILOG_I_ZR_SVR_SCH": 800003,
               "ILOG_I_ZR_SVC_SCH": 800004},
    "tndszd": {"ILOG_I_MP_SVC_SCH": 600004, "ILOG_I_ZR_SVR_WKR": 800001,
               "ILOG_I_ZR_SVC_WKR": 800002, "ILOG_I_ZR_SVR_SCH": 800003,
               "ILOG_I_ZR_SVC_SCH": 800004},
}


@pytest.mark.parametrize("mod", sorted(SURFACE))
def test_module_and_names_exist(mod):
    m = importlib.import_module("necklace_b200" + ("." + mod if mod else ""))
    missing = [n for n in SURFACE[mod] if not hasattr(m, n)]
    assert not missing, (mod, missing)


def test_trainer_hook_registration_and_attributes():
    from necklace_b200.trainer.tnoppt import TrainerOPPytorch
    from necklace_b200.trainer.zroppt import TrainerMPOPPytorch
    for when in ("before", "after"):
        for what in ("train", "epoch", "data_batch", "batch", "do_a_batch_grads",
                     "do_a_train_step"):
            assert hasattr(TrainerOPPytorch, f"register_hook_{when}_{what}")
    assert hasattr(TrainerMPOPPytorch, "get_whole_net_cpu")


def test_log_channels_have_the_reference_numbers_and_switch_service_lines_on(capsys):
    from necklace_b200.rpc import ilog
    from necklace_b200.trainer import service
    for mod, names in CHANNELS.items():
        m = importlib.import_module("necklace_b200.trainer." + mod)
        for name, val in names.items():
            assert getattr(m, name) == val, (mod, name)
    service._dbg("svr_wkr", "hidden")
    assert capsys.readouterr().out == ""
    from necklace_b200.trainer import tndszd
    ilog.il_add(tndszd.ILOG_I_ZR_SVR_WKR)
    try:
        service._dbg("svr_wkr", "shown")
        assert "shown" in capsys.readouterr().out
    finally:
        ilog.il_del(tndszd.ILOG_I_ZR_SVR_WKR)


def test_two_way_group_map_has_the_reference_layout():
    """8 ranks, model parallel 2: mp groups are adjacent pairs, dp groups stride over them
    (reference: necklace/cuda/ncclpgs.py:189-258)."""
    from necklace_b200.comm import groups as G
    from necklace_b200.cuda import ncclpgs
    G.reset_nccl_groups_map()
    try:
        ncclpgs.init_nccl_groups_map(8, 5, 2, 4, True)
        grp = ncclpgs.get_nccl_groups_map_grp_dict()
        assert grp["mp_group"] == [[0, 1], [2, 3], [4, 5], [6, 7]]
        assert grp["dp_group"] == [[0, 2, 4, 6], [1, 3, 5, 7]]
        assert ncclpgs.get_nccl_group_dp().pg_ranks == [1, 3, 5, 7]
        assert ncclpgs.get_nccl_group_mp().pg_ranks == [4, 5]
    finally:
        G.reset_nccl_groups_map()


def test_array_level_helpers_on_a_single_rank_group():
    import ctypes

    import numpy as np
    import torch

    from necklace_b200.comm.symm import TorchGroup
    from necklace_b200.cuda import nbutils, ncclutils
    nc = TorchGroup()
    a = torch.arange(8, dtype=torch.float32)
    assert ncclutils.nccl_all_reduce(a, nc, 1) is a
    outs = torch.zeros(8)
    ncclutils.nccl_all_gather(a, outs, nc, 1)
    assert torch.equal(outs, a)
    assert ncclutils.nccl_all_reduce(None, nc, 1) is None
    assert ncclutils.tensor_size(np.ones((2, 3))) == 6
    assert ncclutils.tensor_dtype(np.ones(2, dtype=np.float16)) == torch.float16
    assert ncclutils.tensor_data_ptr(a) == a.data_ptr()
    assert ncclutils.tensor_data_ptr(np.ones(2)) != 0
    d = nbutils.cuda_to_device(np.ones(3, dtype=np.float32))
    assert isinstance(nbutils.cuda_devarr_c_void_p(d), ctypes.c_void_p)
    assert nbutils.cuda_current_context().type in ("cpu", "cuda")


def test_operator_convenience_methods():
    import torch
    from necklace_b200.trainer.ppoppt import TrainerMPOPPytorch as PP
    from necklace_b200.trainer.tnoppt import TrainerOPPytorch
    from necklace_b200.trainer.zroppt import TrainerMPOPPytorch as ZR
    for name in ("to_ctx", "try_to_ctx", "to_list", "cuda_sync", "check_if_last_batch",
                 "clear_train_data", "train_loop", "metric_log", "init_train_data_it"):
        assert hasattr(TrainerOPPytorch, name), name
    for cls in (PP, ZR):
        assert hasattr(cls, "is_first_part") and hasattr(cls, "is_last_part")
    assert hasattr(ZR, "opts_zero_grad")
    t = TrainerOPPytorch({"ctx": torch.device("cpu"), "net": torch.nn.Linear(2, 2)})
    x = t.to_ctx([torch.ones(2), (torch.zeros(1),)])
    assert isinstance(x, list) and isinstance(x[1], tuple) and x[0].device.type == "cpu"
    assert t.try_to_ctx("text") == "text" and t.to_list(3) == [3] and t.to_list((1, 2)) == [1, 2]
    t.cuda_sync()
    assert t.check_if_last_batch() is False


def test_import_alias_for_scripts_written_against_the_reference(tmp_path):
    """``necklace_b200.compat.install()``: ``import necklace...`` resolves to the modules of this
    package (same objects).  Run in a child process so that the alias does not leak."""
    import subprocess
    import sys
    root = __import__("os").path.dirname(__import__("os").path.dirname(__file__))
    script = tmp_path / "s.py"
    script.write_text(
        "import sys\n"
        f"sys.path.insert(0, {root!r})\n"
        "import necklace_b200.compat as c\n"
        "assert c.install()\n"
        "import necklace\n"
        "from necklace.trainer import tndszd\n"
        "from necklace.cuda import ncclgrp, ncclfns\n"
        "from necklace.frmwrk.pytorch.mpnn import layers\n"
        "from necklace.utils.argutils import attach_nk_args_parser\n"
        "import necklace_b200.trainer.tndszd as real\n"
        "assert tndszd is real and necklace.init is sys.modules['necklace_b200'].init\n"
        "try:\n    import necklace.nothing_here\nexcept ImportError:\n    pass\n"
        "else:\n    raise SystemExit('a missing module resolved')\n"
        "c.uninstall()\n"
        "assert 'necklace.trainer' not in sys.modules\n"
        "print('alias ok')\n")
    r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "alias ok" in r.stdout, r.stderr[-1500:]


def test_alias_path_needs_no_edit_and_reaches_spawned_processes(tmp_path):
    """``PYTHONPATH=$(python -m necklace_b200.compat --path)``: ``import necklace`` is this package
    in the main process and in a process it spawns."""
    import os
    import subprocess
    import sys
    from necklace_b200 import compat
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "s.py"
    script.write_text(
        "import multiprocessing as mp\n\n\n"
        "def child(q):\n"
        "    from necklace.rpc import ilog\n"
        "    import necklace_b200.rpc.ilog as r\n"
        "    q.put(ilog is r)\n\n\n"
        "if __name__ == '__main__':\n"
        "    import necklace\n"
        "    from necklace.trainer import tndszd\n"
        "    import necklace_b200\n"
        "    import necklace_b200.trainer.tndszd as real\n"
        "    assert necklace is necklace_b200 and tndszd is real\n"
        "    ctx = mp.get_context('spawn')\n"
        "    q = ctx.Queue()\n"
        "    p = ctx.Process(target=child, args=(q,))\n"
        "    p.start()\n"
        "    assert q.get(timeout=120) is True\n"
        "    p.join()\n"
        "    print('alias path ok')\n")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([compat.alias_path(), root]))
    r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=300,
                       env=env, cwd=str(tmp_path))
    assert r.returncode == 0 and "alias path ok" in r.stdout, r.stderr[-1500:]
    out = subprocess.run([sys.executable, "-m", "necklace_b200.compat", "--path"],
                         capture_output=True, text=True, cwd=root, timeout=120)
    assert out.stdout.strip() == compat.alias_path()
