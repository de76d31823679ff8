"""Parameter files in nnabla's `.protobuf` format (nn.save_parameters / nn.load_parameters): the hand-written
wire-format writer and reader of nnabla_b200.parametric_functions against google.protobuf itself, with the
message layout of src/nbla/proto/nnabla.proto.tmpl (NNablaProtoBuf.parameter = 200; Parameter.variable_name = 1,
.shape = 20, .data = 100, .need_grad = 101; Shape.dim = 1)."""
import numpy as np
import pytest
import torch
from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

from nnabla_b200 import parametric_functions as PF


def nnabla_messages():
    """The three messages a parameter file uses, declared with the reference's field numbers."""
    fd = descriptor_pb2.FileDescriptorProto(name="nnabla_parameters_subset.proto", package="nbsubset", syntax="proto3")
    T = descriptor_pb2.FieldDescriptorProto
    shape = fd.message_type.add(name="Shape")
    shape.field.add(name="dim", number=1, type=T.TYPE_INT64, label=T.LABEL_REPEATED)
    par = fd.message_type.add(name="Parameter")
    par.field.add(name="variable_name", number=1, type=T.TYPE_STRING, label=T.LABEL_OPTIONAL)
    par.field.add(name="shape", number=20, type=T.TYPE_MESSAGE, label=T.LABEL_OPTIONAL, type_name=".nbsubset.Shape")
    par.field.add(name="data", number=100, type=T.TYPE_FLOAT, label=T.LABEL_REPEATED)
    par.field.add(name="need_grad", number=101, type=T.TYPE_BOOL, label=T.LABEL_OPTIONAL)
    top = fd.message_type.add(name="NNablaProtoBuf")
    top.field.add(name="version", number=1, type=T.TYPE_STRING, label=T.LABEL_OPTIONAL)
    top.field.add(name="parameter", number=200, type=T.TYPE_MESSAGE, label=T.LABEL_REPEATED,
                  type_name=".nbsubset.Parameter")
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    return message_factory.GetMessageClass(pool.FindMessageTypeByName("nbsubset.NNablaProtoBuf"))


@pytest.fixture
def registry():
    PF.set_device("cpu")
    PF.clear_parameters()
    yield PF
    PF.clear_parameters()
    PF._device = None


def some_parameters(rng):
    return {"conv1/bwn_conv/W": rng.randn(4, 3, 3, 3).astype(np.float32),
            "conv1/bwn_conv/Wb": np.sign(rng.randn(4, 3, 3, 3)).astype(np.float32),
            "conv1/bwn_conv/alpha": rng.rand(4).astype(np.float32),
            "conv1/bwn_conv/b": np.float32([0.0, -0.0, 1e-45, 3.4e38]),
            "bn/mean": rng.randn(1, 4, 1, 1).astype(np.float32),
            "fc/inq_affine/I": (rng.rand(5, 7) < 0.5).astype(np.float32),
            "scalar": np.full((), 2.5, np.float32)}


def test_written_file_parses_with_protobuf(registry, tmp_path):
    want = some_parameters(np.random.RandomState(0))
    for k, v in want.items():
        PF.get_parameters()[k] = torch.from_numpy(v)
    path = str(tmp_path / "params.protobuf")
    PF.save_parameters(path)
    msg = nnabla_messages()()
    msg.ParseFromString(open(path, "rb").read())
    assert [p.variable_name for p in msg.parameter] == list(want)
    for p in msg.parameter:
        a = want[p.variable_name]
        assert tuple(p.shape.dim) == a.shape
        assert np.array_equal(np.float32(list(p.data)).view(np.uint32), a.ravel().view(np.uint32))
        assert p.need_grad == (p.variable_name.rsplit("/", 1)[-1] not in ("Wb", "alpha", "mean", "var", "I"))


@pytest.mark.parametrize("packed", [True, False])
def test_protobuf_written_file_loads(registry, tmp_path, packed):
    want = some_parameters(np.random.RandomState(1))
    msg = nnabla_messages()(version="0.1")
    for k, v in want.items():
        p = msg.parameter.add(variable_name=k, need_grad=k.endswith("W"))
        p.shape.dim.extend(v.shape)
        p.data.extend(v.ravel().tolist())
    raw = msg.SerializeToString()
    if not packed:  # an old writer: one field per float (wire type 5), one varint per dimension
        out = bytearray(PF._field(1, 2, b"0.1"))
        for k, v in want.items():
            body = PF._field(1, 2, k.encode())
            body += PF._field(20, 2, b"".join(PF._field(1, 0, PF._varint(d)) for d in v.shape))
            body += b"".join(PF._field(100, 5, np.float32(x).tobytes()) for x in v.ravel())
            if k.endswith("W"):
                body += PF._field(101, 0, PF._varint(1))
            out += PF._field(200, 2, body)
        raw = bytes(out)
        check = nnabla_messages()()
        check.ParseFromString(raw)  # what this test wrote by hand is valid protobuf too
        assert len(check.parameter) == len(want)
    path = str(tmp_path / "theirs.protobuf")
    open(path, "wb").write(raw)
    flags = PF.load_parameters(path)
    got = PF.get_parameters()
    assert list(got) == list(want)
    for k, v in want.items():
        assert tuple(got[k].shape) == v.shape and got[k].dtype == torch.float32
        assert np.array_equal(got[k].numpy().view(np.uint32), v.view(np.uint32))
        assert flags[k] == k.endswith("W")


def test_round_trip_and_errors(registry, tmp_path):
    want = some_parameters(np.random.RandomState(2))
    for k, v in want.items():
        PF.get_parameters()[k] = torch.from_numpy(v)
    path = str(tmp_path / "p.protobuf")
    PF.save_parameters(path)
    PF.clear_parameters()
    PF.load_parameters(path)
    for k, v in want.items():
        assert np.array_equal(PF.get_parameters()[k].numpy().view(np.uint32), v.view(np.uint32))
    with pytest.raises(ValueError):
        PF.save_parameters(str(tmp_path / "p.h5"))
    open(str(tmp_path / "cut.protobuf"), "wb").write(open(path, "rb").read()[:-3])
    with pytest.raises(ValueError):
        PF.load_parameters(str(tmp_path / "cut.protobuf"))
