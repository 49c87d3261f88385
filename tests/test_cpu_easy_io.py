"""Unified file API, object store, image VAE wrappers (CPU)."""
import io

import numpy as np
import pytest
import torch

from cosmos_predict25_b200.utils.easy_io import Boto3Backend, easy_io
from cosmos_predict25_b200.utils.object_store import ObjectStore


def test_roundtrip_formats(tmp_path):
    objs = {"a.json": {"x": [1, 2], "y": np.float32(1.5)}, "b.yaml": {"k": "v"}, "c.pkl": {"t": (1, 2)}, "d.txt": "hello",
            "e.jsonl": [{"i": 1}, {"i": 2}], "f.csv": [["a", "b"], ["1", "2"]]}
    for name, obj in objs.items():
        p = str(tmp_path / "sub" / name)
        easy_io.dump(obj, p)
        back = easy_io.load(p)
        if name == "a.json":
            assert back == {"x": [1, 2], "y": 1.5}
        else:
            assert back == obj
    t = {"w": torch.arange(4.0)}
    easy_io.dump(t, str(tmp_path / "w.pt"))
    assert torch.equal(easy_io.load(str(tmp_path / "w.pt"))["w"], t["w"])
    easy_io.dump(np.arange(5), str(tmp_path / "n.npy"))
    assert np.array_equal(easy_io.load(str(tmp_path / "n.npy")), np.arange(5))
    img = (np.random.rand(8, 8, 3) * 255).astype(np.uint8)
    easy_io.dump(img, str(tmp_path / "i.png"))
    assert np.array_equal(easy_io.load(str(tmp_path / "i.png"), fmt="np"), img)
    easy_io.dump({"m.txt": b"abc"}, str(tmp_path / "t.tar"))
    tf = easy_io.load(str(tmp_path / "t.tar"))
    assert tf.extractfile("m.txt").read() == b"abc"
    assert easy_io.dump({"a": 1}, file_format="json") == '{"a": 1}'
    with pytest.raises(TypeError):
        easy_io.load(str(tmp_path / "x.unknownext"))


def test_local_fs_ops(tmp_path):
    d = tmp_path / "d"
    easy_io.put_text("x", str(d / "a" / "1.txt"))
    easy_io.put(b"y", str(d / "2.bin"))
    assert easy_io.exists(str(d / "2.bin")) and easy_io.isdir(str(d / "a")) and easy_io.isfile(str(d / "a" / "1.txt"))
    assert sorted(easy_io.list_dir_or_file(str(d), list_dir=False, recursive=True)) == ["2.bin", "a/1.txt"]
    assert list(easy_io.list_dir_or_file(str(d), list_file=False)) == ["a"]
    assert list(easy_io.list_dir_or_file(str(d), list_dir=False, suffix=".txt", recursive=True)) == ["a/1.txt"]
    easy_io.copyfile(str(d / "2.bin"), str(d / "3.bin"))
    assert easy_io.get(str(d / "3.bin")) == b"y"
    with easy_io.get_local_path(str(d / "3.bin")) as p:
        assert open(p, "rb").read() == b"y"
    easy_io.remove(str(d / "3.bin"))
    assert not easy_io.exists(str(d / "3.bin"))
    assert easy_io.join_path(str(d), "a", "b") == str(d / "a" / "b")
    assert easy_io._parse_uri_prefix("s3://b/k") == "s3" and easy_io._parse_uri_prefix("/x/y") == "" and easy_io._parse_uri_prefix("c:s3://b") == "s3"


class _FakeS3:
    def __init__(self):
        self.store = {}

    def upload_fileobj(self, f, b, k): self.store[(b, k)] = f.read()
    def download_fileobj(self, b, k, buf): buf.write(self.store[(b, k)])

    def head_object(self, Bucket, Key):
        if (Bucket, Key) not in self.store:
            raise KeyError(Key)

    def list_objects_v2(self, Bucket, Prefix, MaxKeys=1000):
        return {"KeyCount": sum(1 for (b, k) in self.store if b == Bucket and k.startswith(Prefix))}

    def delete_object(self, Bucket, Key): self.store.pop((Bucket, Key))


def test_s3_backend_against_fake_client():
    fake = _FakeS3()
    easy_io.backend_instances["s3"] = Boto3Backend(client=fake, path_mapping={"s3://alias/": "s3://real/"})
    try:
        easy_io.dump({"a": 1}, "s3://alias/dir/o.json")
        assert ("real", "dir/o.json") in fake.store
        assert easy_io.load("s3://real/dir/o.json") == {"a": 1}
        assert easy_io.exists("s3://real/dir/o.json") and easy_io.isdir("s3://real/dir") and not easy_io.exists("s3://real/none")
        easy_io.remove("s3://real/dir/o.json")
        assert not fake.store
    finally:
        easy_io.backend_instances.pop("s3")


def test_object_store_local(tmp_path):
    st = ObjectStore(root=str(tmp_path))
    st.save_object({"a": torch.ones(2)}, "ck/x.pt", type="torch")
    st.save_object({"b": 2}, "ck/y.json", type="json")
    assert st.object_exists("ck/x.pt") and torch.equal(st.load_object("ck/x.pt")["a"], torch.ones(2))
    assert st.load_object("ck/y.json", type="json") == {"b": 2}
    assert sorted(st.list_objects("ck")) == ["x.pt", "y.json"]
    st.delete_object("ck/y.json")
    assert not st.object_exists("ck/y.json")


def test_image_vae_wrappers(tmp_path):
    from cosmos_predict25_b200.models.image_vae import SDVAE, StateDictVAE

    class Tiny(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.encoder = torch.nn.Conv2d(3, 4, 8, stride=8)
            self.decoder = torch.nn.ConvTranspose2d(4, 3, 8, stride=8)

    src = Tiny()
    torch.save(src.encoder.state_dict(), tmp_path / "enc.pt")
    torch.save(src.decoder.state_dict(), tmp_path / "dec.pt")
    easy_io.dump((torch.full((4,), 0.5), torch.full((4,), 2.0)), str(tmp_path / "ms.pt"))
    vae = StateDictVAE(str(tmp_path / "enc.pt"), str(tmp_path / "dec.pt"), Tiny(), "tiny", str(tmp_path / "ms.pt"), latent_ch=4, is_bf16=False)
    x = torch.randn(1, 3, 16, 16)
    z = vae.encode(x)
    assert torch.allclose(z, (src.encoder(x) - 0.5) / 2.0, atol=1e-5)
    assert torch.allclose(vae.decode(z), src.decoder(src.encoder(x)), atol=1e-4)

    class FakeKL(torch.nn.Module):
        def encode(self, x):
            m = torch.nn.functional.avg_pool2d(x, 8)
            m = torch.cat([m, m[:, :1]], 1)
            return {"latent_dist": type("D", (), {"mean": m, "std": torch.ones_like(m)})()}

        def decode(self, z):
            return {"sample": torch.nn.functional.interpolate(z[:, :3], scale_factor=8)}

    sd = SDVAE(vae=FakeKL(), dtype=torch.float32)
    img = torch.rand(2, 3, 32, 32) * 2 - 1
    lat = sd.encode(img)
    assert lat.shape == (2, 4, 2, 2) and sd.decode(lat).shape == img.shape
