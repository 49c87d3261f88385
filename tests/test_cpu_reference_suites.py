"""The reference's own unit-test files, run unmodified against this package (module names mapped by
``reference_alias_plugin``). Each entry: test file inside the reference tree, the mapping, and the tests of that file that are
expected to pass (all of them unless a reason is given)."""

import json
import os
import subprocess
import sys

import pytest

from reference_oracle import reference_dir

_HERE = os.path.dirname(os.path.abspath(__file__))
P = "cosmos_predict25_b200"
def _offline_checkpoint_cache(tmp_path):
    """No network here: the two checkpoints those tests resolve are placed in the local cache directory."""
    root = tmp_path / "cache"
    (root / "7219c6c7-f878-4137-bbdb-76842ea85e70").mkdir(parents=True)
    (root / "685afcaa-4de2-42fe-b7b9-69f7a2dee4d8").write_bytes(b"0")
    return {"COSMOS_CHECKPOINT_DIR": str(root)}


def _single_rank_on_the_host(tmp_path):
    """The data-parallel checkpointer test as one gloo rank writing under the temporary directory."""
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    return {"COSMOS_ALIAS_NO_CUDA": "1", "IMAGINAIRE_OUTPUT_ROOT": str(tmp_path / "out"), "RANK": "0", "WORLD_SIZE": "1", "LOCAL_RANK": "0",
            "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)}


def _tiny_t5_checkpoint(tmp_path):
    """No network here: a one-layer random T5 encoder of the real width (1024) with a sentencepiece model trained on a few
    sentences stands in for the 11B checkpoint; shapes, padding, truncation and caching are what those tests check."""
    import sentencepiece as spm
    from transformers import T5Config, T5EncoderModel, T5TokenizerFast
    d = tmp_path / "t5"
    d.mkdir()
    (d / "corpus.txt").write_text("\n".join(["this is a test prompt", "first second third prompt", "testing global encoder",
                                             "this is a very long prompt", "short prompt"] * 20))
    spm.SentencePieceTrainer.train(input=str(d / "corpus.txt"), model_prefix=str(d / "spiece"), vocab_size=60, model_type="unigram",
                                   pad_id=0, eos_id=1, unk_id=2, bos_id=-1, hard_vocab_limit=False, minloglevel=2)
    T5TokenizerFast(vocab_file=str(d / "spiece.model"), extra_ids=0).save_pretrained(str(d))
    T5EncoderModel(T5Config(vocab_size=64, d_model=1024, d_kv=16, num_heads=2, d_ff=64, num_layers=1, feed_forward_proj="relu")).save_pretrained(str(d))
    return {"COSMOS_T5_MODEL_DIR": str(d)}


PREPARE = {"checkpoint_db_test.py": _offline_checkpoint_cache, "ddp_test.py": _single_rank_on_the_host, "get_t5_emb_test.py": _tiny_t5_checkpoint}
# tests the reference marks "run manually" that do run here: the mark is dropped from the copy
UNSKIP = {"ddp_test.py": ["test_checkpointer_local"]}
SUITES = [
    ("cosmos_predict2/_src/imaginaire/modules/camera_test.py", {"cosmos_predict2._src.imaginaire.modules.camera": f"{P}.modules.camera"}, ""),
    ("cosmos_predict2/_src/imaginaire/utils/validator_test.py",
     {"cosmos_predict2._src.imaginaire.utils.validator": f"{P}.utils.validator",
      "cosmos_predict2._src.imaginaire.utils.validator_params": f"{P}.utils.validator_params"}, ""),
    ("cosmos_predict2/_src/imaginaire/datasets/mock_dataset_test.py",
     {"cosmos_predict2._src.imaginaire.datasets.mock_dataset": f"{P}.data.mock", "cosmos_predict2._src.imaginaire.lazy_config": f"{P}.utils.lazy_config"}, ""),
    ("cosmos_predict2/_src/predict2/datasets/cached_replay_dataloader_test.py",
     {"cosmos_predict2._src.predict2.datasets.cached_replay_dataloader": f"{P}.data.loaders"}, ""),
    ("cosmos_predict2/_src/predict2/datasets/decoders/video_decoder_test.py",
     {"cosmos_predict2._src.predict2.datasets.decoders.video_decoder": f"{P}.data.video_decoder"}, ""),
    ("cosmos_predict2/_src/predict2/configs/text2world/config_test.py",
     {"cosmos_predict2._src.imaginaire.utils.config_helper": f"{P}.utils.config",
      "cosmos_predict2._src.predict2.configs.text2world.config": f"{P}.configs.text2world"}, ""),
    ("cosmos_predict2/_src/imaginaire/utils/ema_test.py",
     {"cosmos_predict2._src.imaginaire.model": f"{P}.trainer.model", "cosmos_predict2._src.imaginaire.utils.ema": f"{P}.utils.ema"},
     ""),
    ("cosmos_predict2/_src/imaginaire/datasets/webdataset/distributors/multi_aspect_ratio_v2_test.py",
     {"cosmos_predict2._src.imaginaire.config": f"{P}.utils.config", "cosmos_predict2._src.imaginaire.utils": f"{P}.utils",
      "cosmos_predict2._src.imaginaire.datasets.webdataset.config.schema": f"{P}.data.webdataset",
      "cosmos_predict2._src.imaginaire.datasets.webdataset.distributors.multi_aspect_ratio_v2": f"{P}.data.webdataset"}, ""),
    ("cosmos_predict2/_src/imaginaire/checkpointer/ddp_test.py",
     {"cosmos_predict2._src.imaginaire.checkpointer.ddp": f"{P}.checkpoint.ddp", "cosmos_predict2._src.imaginaire.config": f"{P}.utils.config",
      "cosmos_predict2._src.imaginaire.lazy_config": f"{P}.utils.lazy_config", "cosmos_predict2._src.imaginaire.model": f"{P}.trainer.model",
      "cosmos_predict2._src.imaginaire.trainer": f"{P}.trainer.trainer", "cosmos_predict2._src.imaginaire.utils.distributed": f"{P}.utils.distributed",
      "cosmos_predict2._src.imaginaire.utils.log": f"{P}.utils.log", "megatron.core.parallel_state": f"{P}.parallel.parallel_state"},
     "test_checkpointer_local"),
    ("cosmos_predict2/_src/predict2/inference/get_t5_emb_test.py",
     {"cosmos_predict2._src.predict2.inference.get_t5_emb": f"{P}.pipeline.get_t5_emb"}, ""),
    ("cosmos_predict2/config_test.py", {"cosmos_predict2.config": f"{P}.config"}, ""),
    ("cosmos_predict2/_src/imaginaire/utils/misc_test.py", {"cosmos_predict2._src.imaginaire.utils.misc": f"{P}.utils.misc"}, ""),
    ("cosmos_predict2/_src/imaginaire/utils/checkpoint_db_test.py",
     {"cosmos_predict2._src.imaginaire.utils.checkpoint_db": f"{P}.utils.checkpoint_db"}, "not hf_ and not all_checkpoints"),     # the L1 tests download from the hub
]


@pytest.mark.parametrize("path,aliases,select", SUITES, ids=[s[0].split("/")[-1] for s in SUITES])
def test_reference_test_file_passes_against_this_package(path, aliases, select, tmp_path):
    root = reference_dir()
    if root is None:
        pytest.skip("no copy of the reference implementation here")
    src = os.path.join(root, path)
    # a copy outside the reference tree: its pyproject / conftest must not configure the run, its packages must not be importable
    dst = tmp_path / os.path.basename(path)
    text = open(src).read()
    for name in UNSKIP.get(os.path.basename(path), []):
        head, sep, tail = text.partition(f"def {name}(")
        lines = head.rstrip("\n").split("\n")
        assert sep and lines[-1].startswith("@pytest.mark.skip"), name
        text = "\n".join(lines[:-1]) + "\n" + sep + tail
    dst.write_text(text)
    (tmp_path / "pytest.ini").write_text("[pytest]\n")
    extra = PREPARE.get(os.path.basename(path), lambda _: {})(tmp_path)
    env = dict(os.environ, **extra, COSMOS_ALIAS_JSON=json.dumps(aliases), PYTHONPATH=os.pathsep.join([_HERE, os.path.dirname(_HERE)]))
    cmd = [sys.executable, "-m", "pytest", str(dst), "-q", "-x", "-p", "reference_alias_plugin", "-p", "no:cacheprovider", "--rootdir", str(tmp_path)]
    if select:
        cmd += ["-k", select]
    out = subprocess.run(cmd, env=env, cwd=str(tmp_path), capture_output=True, text=True, timeout=600)
    tail = (out.stdout + out.stderr)[-3000:]
    assert out.returncode == 0, tail
    assert " passed" in out.stdout, tail
