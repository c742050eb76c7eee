"""ONNX files for the import tests, serialised by the protobuf runtime.

The ``onnx`` package is not installed where these tests run, so the handful of messages a model
needs are declared here (names and field numbers of the public ``onnx.proto``) and encoded by
``google.protobuf``; the importer under test decodes them with its own wire-format reader, so
writer and reader are two independent implementations of the format."""
import numpy as np
from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

_F = descriptor_pb2.FieldDescriptorProto
_T = {"int64": _F.TYPE_INT64, "int32": _F.TYPE_INT32, "float": _F.TYPE_FLOAT, "string": _F.TYPE_STRING,
      "bytes": _F.TYPE_BYTES, "double": _F.TYPE_DOUBLE}


def _build():
    fd = descriptor_pb2.FileDescriptorProto(name="onnx_subset.proto", package="onnx_subset", syntax="proto2")

    def msg(name, fields):
        m = fd.message_type.add(name=name)
        for fname, num, ftype, rep in fields:
            f = m.field.add(name=fname, number=num,
                            label=_F.LABEL_REPEATED if rep else _F.LABEL_OPTIONAL)
            if ftype in _T:
                f.type = _T[ftype]
                # as in onnx.proto (proto2): only the tensor payload fields are packed; dims and the
                # attribute lists are one key per element
                if rep and fname in ("float_data", "int32_data", "int64_data"):
                    f.options.packed = True
            else:
                f.type = _F.TYPE_MESSAGE
                f.type_name = ".onnx_subset." + ftype

    msg("TensorProto", [("dims", 1, "int64", True), ("data_type", 2, "int32", False),
                        ("float_data", 4, "float", True), ("int32_data", 5, "int32", True),
                        ("int64_data", 7, "int64", True), ("name", 8, "string", False),
                        ("raw_data", 9, "bytes", False)])
    msg("AttributeProto", [("name", 1, "string", False), ("f", 2, "float", False), ("i", 3, "int64", False),
                           ("s", 4, "bytes", False), ("t", 5, "TensorProto", False),
                           ("floats", 7, "float", True), ("ints", 8, "int64", True),
                           ("type", 20, "int32", False)])
    msg("NodeProto", [("input", 1, "string", True), ("output", 2, "string", True), ("name", 3, "string", False),
                      ("op_type", 4, "string", False), ("attribute", 5, "AttributeProto", True)])
    msg("Dimension", [("dim_value", 1, "int64", False), ("dim_param", 2, "string", False)])
    msg("TensorShapeProto", [("dim", 1, "Dimension", True)])
    msg("TensorTypeProto", [("elem_type", 1, "int32", False), ("shape", 2, "TensorShapeProto", False)])
    msg("TypeProto", [("tensor_type", 1, "TensorTypeProto", False)])
    msg("ValueInfoProto", [("name", 1, "string", False), ("type", 2, "TypeProto", False)])
    msg("GraphProto", [("node", 1, "NodeProto", True), ("name", 2, "string", False),
                       ("initializer", 5, "TensorProto", True), ("input", 11, "ValueInfoProto", True),
                       ("output", 12, "ValueInfoProto", True)])
    msg("OperatorSetIdProto", [("domain", 1, "string", False), ("version", 2, "int64", False)])
    msg("ModelProto", [("ir_version", 1, "int64", False), ("producer_name", 2, "string", False),
                       ("graph", 7, "GraphProto", False), ("opset_import", 8, "OperatorSetIdProto", True)])
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    get = getattr(message_factory, "GetMessageClass", None)
    if get is None:  # older protobuf runtimes
        factory = message_factory.MessageFactory(pool)
        get = factory.GetPrototype
    return {n: get(pool.FindMessageTypeByName("onnx_subset." + n))
            for n in ("TensorProto", "AttributeProto", "NodeProto", "ValueInfoProto", "GraphProto", "ModelProto")}


_M = _build()
FLOAT, INT64, FLOAT16 = 1, 7, 10


def tensor(name, arr, raw=False):
    arr = np.asarray(arr)
    t = _M["TensorProto"](name=name, dims=list(arr.shape))
    if arr.dtype == np.float32:
        t.data_type = FLOAT
        if raw:
            t.raw_data = arr.astype("<f4").tobytes()
        else:
            t.float_data.extend(float(v) for v in arr.ravel())
    elif arr.dtype == np.int64:
        t.data_type = INT64
        t.int64_data.extend(int(v) for v in arr.ravel())
    else:
        raise TypeError(arr.dtype)
    return t


def node(op_type, inputs, outputs, **attrs):
    n = _M["NodeProto"](op_type=op_type, input=list(inputs), output=list(outputs))
    for k, v in attrs.items():
        a = n.attribute.add(name=k)
        if isinstance(v, float):
            a.f, a.type = v, 1
        elif isinstance(v, int):
            a.i, a.type = v, 2
        elif isinstance(v, bytes):
            a.s, a.type = v, 3
        elif isinstance(v, np.ndarray):
            a.t.CopyFrom(tensor("", v))
            a.type = 4
        elif isinstance(v, (list, tuple)) and all(isinstance(e, int) for e in v):
            a.ints.extend(v)
            a.type = 7
        else:
            raise TypeError(f"attribute {k}: {type(v)}")
    return n


def value_info(name, shape):
    v = _M["ValueInfoProto"](name=name)
    v.type.tensor_type.elem_type = FLOAT
    for d in shape:
        dim = v.type.tensor_type.shape.dim.add()
        if d is None:
            dim.dim_param = "N"
        else:
            dim.dim_value = d
    return v


def model(nodes, inputs, outputs, initializers, list_initializers_as_inputs=False) -> bytes:
    g = _M["GraphProto"](name="g")
    g.node.extend(nodes)
    g.input.extend(inputs)
    if list_initializers_as_inputs:  # what exporters before IR version 4 wrote
        g.input.extend(value_info(t.name, list(t.dims)) for t in initializers)
    g.output.extend(outputs)
    g.initializer.extend(initializers)
    m = _M["ModelProto"](ir_version=7, producer_name="munet_b200_tests", graph=g)
    m.opset_import.add(domain="", version=11)
    return m.SerializeToString()
