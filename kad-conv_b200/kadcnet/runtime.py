"""Inference entry point with the reference's signature.

Mirrors KAD-CNet/inference/runtime.py of the reference project: load_model(...) :30-77 and the
StaticGraph CUDA-graph wrapper :106-131. Backends:
  'raw'        plain PyTorch modules (the definition; any device)
  'optimized'  kadcnet.engine.FastDetector: NHWC, KAD-Conv and 1x1 convolutions on the sm_100a kernels
  'graph'      'optimized' captured in a CUDA graph per input shape
`weights` may be a checkpoint path (a state_dict, or a dict with a 'model'/'ema' entry holding a module or a
state_dict) or None: then the model is built from `config` (a model YAML or None for KAD-CNet-S) and
initialised from `seed`, because no released checkpoint ships with this package.
"""
import torch

from .engine import FastDetector
from .model import DetectionModel


def numerical_protocol():
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cudnn.benchmark = True


def clone_output(value):
    if isinstance(value, torch.Tensor):
        return value.clone()
    if isinstance(value, (list, tuple)):
        return type(value)(clone_output(v) for v in value)
    return value


class StaticGraph:
    """Captures forward(sample) once; each call copies the input in, replays, and (by default) clones the output."""

    def __init__(self, forward, sample, warmup=3):
        self.input = sample.clone()
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.no_grad(), torch.cuda.stream(stream):
            for _ in range(warmup):
                forward(self.input)
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph, stream=stream):
            self.output = forward(self.input)
        torch.cuda.synchronize()

    def __call__(self, value, clone=True):
        from kadconv import ops
        ops.status_poll(self.input.device)          # an earlier replay whose kernel gave up on a wait raises here
        self.input.copy_(value)
        self.graph.replay()
        ops.status_snapshot(self.input.device)
        return clone_output(self.output) if clone else self.output


def graph_forward(forward):
    captures = {}

    def run(value, clone=True):
        key = (tuple(value.shape), value.dtype, value.device)
        if key not in captures:
            captures[key] = StaticGraph(forward, value)
        return captures[key](value, clone=clone)
    return run


def _state_dict_from(checkpoint, key):
    obj = checkpoint
    if isinstance(checkpoint, dict) and ('model' in checkpoint or 'ema' in checkpoint):
        k = key if key != 'auto' else ('ema' if checkpoint.get('ema') is not None else 'model')
        if k not in ('model', 'ema'):
            raise ValueError('Select model or ema checkpoint entry')
        obj = checkpoint.get(k)
        if obj is None:
            raise ValueError('Checkpoint lacks model/ema')
    return obj.state_dict() if hasattr(obj, 'state_dict') else obj


def load_model(weights=None, backend='raw', device='cuda:0', config=None, fuse=True, checkpoint_key='auto',
               dtype=torch.float16, seed=0, state_dict=None, randomize=False, conv3x3='library'):
    if backend not in {'raw', 'optimized', 'graph'}:
        raise ValueError(backend)
    numerical_protocol()
    torch.manual_seed(seed)
    model = DetectionModel(config)
    if state_dict is None and weights is None and randomize:
        randomize_for_benchmark(model, seed)
    if state_dict is not None:
        model.load_state_dict(state_dict)
    elif weights is not None:
        ck = torch.load(weights, map_location='cpu', weights_only=False)
        model.load_state_dict({k: v.float() for k, v in _state_dict_from(ck, checkpoint_key).items()})
    model = model.float().eval()
    if fuse:
        model = model.fuse()
    model = model.to(device).eval()
    if backend == 'raw':
        return model
    if not str(device).startswith('cuda'):
        raise ValueError('Acceleration requires CUDA')
    if not fuse:
        raise ValueError("the 'optimized' and 'graph' backends run the fused model")
    fast = FastDetector(model, dtype=dtype, conv3x3=conv3x3)
    if backend == 'graph':
        fast.forward = graph_forward(fast.forward)
    return fast


def randomize_for_benchmark(model, seed=0, offset_std=0.5, cls_bias=-3.0, cls_gain=60.0):
    """Seeded synthetic weights for a model without a checkpoint. The stock initialisation is degenerate for
    inference measurements: zero offset convolutions (no deformation), identity BatchNorm statistics, and class
    biases so low that NMS receives no candidate. This redraws those tensors in place (call before fuse())."""
    g = torch.Generator().manual_seed(seed)
    head = model.model[-1]
    with torch.no_grad():
        for name, m in model.named_modules():
            if isinstance(m, torch.nn.BatchNorm2d):
                m.running_mean.copy_(torch.randn(m.running_mean.shape, generator=g) * 0.1)
                m.running_var.copy_(torch.rand(m.running_var.shape, generator=g) + 0.5)
                m.weight.copy_(torch.rand(m.weight.shape, generator=g) + 0.5)
                m.bias.copy_(torch.randn(m.bias.shape, generator=g) * 0.1)
            elif name.endswith('conv_offset'):
                fan_in = m.weight[0].numel()
                m.weight.copy_(torch.randn(m.weight.shape, generator=g) * (offset_std / fan_in ** 0.5))
                m.bias.copy_(torch.randn(m.bias.shape, generator=g) * (0.1 * offset_std))
        for seq in head.cv3:
            last = seq[-1]
            last.weight.mul_(cls_gain)
            last.bias.copy_(torch.randn(last.bias.shape, generator=g) * 0.1 + cls_bias)
    return model
