"""ONNX-JSON export / import of feed-forward models.

The document schema is the reference's (scirust-onnx/src/lib.rs:28-112): ``{name, ir_version: 7,
producer_name, producer_version, domain: "ai.scirust", model_version, doc_string, graph: {name, inputs,
outputs, nodes, initializers}}`` with value infos ``{name, elem_type: 1, shape: {dims: [{dim_value,
dim_param}]}}``, nodes ``{op_type, inputs, outputs, attributes: [{name, type, i|ints|f|s}], name}`` and
initializers ``{name, dims, data_type: 1, raw_data: [f32...]}``; a symbolic batch is the dim_param
``"batch_size"``. Like the reference's exporter, a ``Linear`` becomes ``Gemm`` (alpha = beta = 1,
transB = 0, weight stored ``[in, out]``) or ``MatMul`` without bias, with parameters named
``param_{i}`` in layer order (lib.rs:115-283).

Beyond the reference (whose exporter assumes Linear/ReLU stacks and whose importer only returns the
weights): the exporter walks the real layer list of a ``Sequential`` (Linear, ReLU, Sigmoid, Tanh, GELU,
SiLU, LayerNorm, Dropout as Identity) and ``run_graph`` evaluates an imported graph, so an
export -> import -> run round trip reproduces the model's outputs.
"""
from __future__ import annotations

import json

import torch
import torch.nn.functional as F

from ..nn import modules as M

PRODUCER = "scirust_b200 ONNX-JSON exporter"


def _dim(v):
    return {"dim_value": None, "dim_param": "batch_size"} if v is None or v < 0 else {"dim_value": int(v),
                                                                                     "dim_param": None}


def _attr(name, value):
    if isinstance(value, bool) or isinstance(value, int):
        return {"name": name, "type": "INT", "i": int(value)}
    if isinstance(value, float):
        return {"name": name, "type": "FLOAT", "f": float(value)}
    if isinstance(value, str):
        return {"name": name, "type": "STRING", "s": value}
    return {"name": name, "type": "INTS", "ints": [int(v) for v in value]}


def _tensor(name, t: torch.Tensor):
    t = t.detach().float().cpu()
    return {"name": name, "dims": [int(d) for d in t.shape], "data_type": 1, "raw_data": t.reshape(-1).tolist()}


_ACTIVATIONS = {M.ReLU: "Relu", M.Sigmoid: "Sigmoid", M.Tanh: "Tanh", M.GELU: "Gelu", M.SiLU: "Swish",
                M.Dropout: "Identity"}


def export_sequential(model, model_name: str, input_shape=(-1, None), version: str = "0.1.0") -> str:
    """Serialise a ``Sequential`` (or a single layer) to an ONNX-JSON string. ``input_shape`` is
    ``(batch, features)``; a negative batch is symbolic."""
    layers = list(model.layers) if isinstance(model, M.Sequential) else [model]
    nodes, inits = [], []
    prev, n_param, feat = "input", 0, input_shape[1]
    if feat is None:
        first = next((l for l in layers if isinstance(l, M.Linear)), None)
        if first is None:
            raise ValueError("input feature count needed when the model has no Linear layer")
        feat = first.in_features
    in_feat = feat
    for i, l in enumerate(layers):
        out = f"t{i}"
        if isinstance(l, M.Linear):
            w = f"param_{n_param}"
            inits.append(_tensor(w, l.weight))
            n_param += 1
            if l.bias is not None:
                b = f"param_{n_param}"
                inits.append(_tensor(b, l.bias.reshape(-1)))
                n_param += 1
                nodes.append({"op_type": "Gemm", "inputs": [prev, w, b], "outputs": [out],
                              "attributes": [_attr("alpha", 1.0), _attr("beta", 1.0), _attr("transB", 0)],
                              "name": f"fc{i}"})
            else:
                nodes.append({"op_type": "MatMul", "inputs": [prev, w], "outputs": [out], "attributes": [],
                              "name": f"fc{i}"})
            feat = l.out_features
        elif isinstance(l, M.LayerNorm):
            g, b = f"param_{n_param}", f"param_{n_param + 1}"
            params = [p for p in l.parameters()]
            inits += [_tensor(g, params[0].reshape(-1)), _tensor(b, params[1].reshape(-1))]
            n_param += 2
            nodes.append({"op_type": "LayerNormalization", "inputs": [prev, g, b], "outputs": [out],
                          "attributes": [_attr("axis", -1), _attr("epsilon", float(getattr(l, "eps", 1e-5)))],
                          "name": f"ln{i}"})
        elif type(l) in _ACTIVATIONS:
            nodes.append({"op_type": _ACTIVATIONS[type(l)], "inputs": [prev], "outputs": [out], "attributes": [],
                          "name": f"act{i}"})
        else:
            raise ValueError(f"export_sequential: layer {type(l).__name__} has no ONNX-JSON mapping")
        prev = out
    if nodes:
        nodes[-1]["outputs"] = ["output"]
    doc = {
        "name": model_name, "ir_version": 7, "producer_name": PRODUCER, "producer_version": version,
        "domain": "ai.scirust", "model_version": 1, "doc_string": "exported by scirust_b200",
        "graph": {"name": model_name,
                  "inputs": [{"name": "input", "elem_type": 1, "shape": {"dims": [_dim(input_shape[0]), _dim(in_feat)]}}],
                  "outputs": [{"name": "output", "elem_type": 1, "shape": {"dims": [_dim(-1), _dim(feat)]}}],
                  "nodes": nodes, "initializers": inits}}
    return json.dumps(doc, indent=2)


class OnnxGraph:
    """Parsed ONNX-JSON document."""

    def __init__(self, doc: dict):
        for k in ("name", "ir_version", "graph"):
            if k not in doc:
                raise ValueError(f"ONNX-JSON: missing field {k!r}")
        g = doc["graph"]
        for k in ("inputs", "outputs", "nodes", "initializers"):
            if k not in g:
                raise ValueError(f"ONNX-JSON: graph is missing {k!r}")
        self.doc = doc

    @property
    def nodes(self):
        return self.doc["graph"]["nodes"]

    def weights(self):
        """[(name, shape, flat fp32 values)] in initializer order (lib.rs:303)."""
        return [(t["name"], list(t["dims"]), list(t["raw_data"])) for t in self.doc["graph"]["initializers"]]

    def tensors(self) -> dict:
        out = {}
        for t in self.doc["graph"]["initializers"]:
            n = 1
            for d in t["dims"]:
                n *= d
            if n != len(t["raw_data"]):
                raise ValueError(f"initializer {t['name']}: {len(t['raw_data'])} values for dims {t['dims']}")
            out[t["name"]] = torch.tensor(t["raw_data"], dtype=torch.float32).reshape(t["dims"])
        return out


def import_onnx_json(text: str) -> OnnxGraph:
    return OnnxGraph(json.loads(text))


def _attrs(node) -> dict:
    out = {}
    for a in node.get("attributes", []):
        out[a["name"]] = a.get("i", a.get("f", a.get("s", a.get("ints"))))
    return out


def run_graph(graph: OnnxGraph, x: torch.Tensor) -> torch.Tensor:
    """Evaluate the graph on ``x`` (fp32). Every node input must be the graph input, an initializer or
    an earlier node's output; unknown operators are refused."""
    env = dict(graph.tensors())
    env[graph.doc["graph"]["inputs"][0]["name"]] = x.float()
    for n in graph.nodes:
        try:
            ins = [env[i] for i in n["inputs"]]
        except KeyError as e:
            raise ValueError(f"node {n.get('name')}: dangling input {e}") from None
        op, at = n["op_type"], _attrs(n)
        if op == "Gemm":
            a, b = ins[0], ins[1]
            if at.get("transA", 0):
                a = a.t()
            if at.get("transB", 0):
                b = b.t()
            y = at.get("alpha", 1.0) * (a @ b)
            if len(ins) > 2:
                y = y + at.get("beta", 1.0) * ins[2]
        elif op == "MatMul":
            y = ins[0] @ ins[1]
        elif op == "Add":
            y = ins[0] + ins[1]
        elif op == "Relu":
            y = F.relu(ins[0])
        elif op == "Sigmoid":
            y = torch.sigmoid(ins[0])
        elif op == "Tanh":
            y = torch.tanh(ins[0])
        elif op == "Gelu":
            y = F.gelu(ins[0])
        elif op == "Swish":
            y = F.silu(ins[0])
        elif op == "Identity":
            y = ins[0]
        elif op == "LayerNormalization":
            y = F.layer_norm(ins[0], ins[0].shape[-1:], ins[1], ins[2], at.get("epsilon", 1e-5))
        elif op == "Softmax":
            y = torch.softmax(ins[0], at.get("axis", -1))
        else:
            raise ValueError(f"run_graph: unsupported operator {op}")
        env[n["outputs"][0]] = y
    return env[graph.doc["graph"]["outputs"][0]["name"]]
