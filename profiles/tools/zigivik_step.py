"""One Zigivik step at bench sizes for launch lists / ncu captures: `python profiles/tools/zigivik_step.py decode|prefill [layers]` (3 steps;
the decode variant runs eagerly so that every kernel is a launch of its own)."""
import sys, torch
sys.path.insert(0, __import__('os').path.dirname(__import__('os').path.dirname(__import__('os').path.dirname(__import__('os').path.abspath(__file__)))))
from paligemma_multimodal_system_b200 import bench_seq
from paligemma_multimodal_system_b200.engine import SequenceEngine
mode = sys.argv[1]
layers = int(sys.argv[2]) if len(sys.argv) > 2 else 8
cfg = bench_seq.zigivik_config(2048, 32, 8, 64, 8192, 32000, layers)
model = bench_seq.random_zigivik(cfg)
g = torch.Generator().manual_seed(1)
if mode == 'decode':
    B, ctx = 64, 1024
    eng = SequenceEngine(model, B * (ctx + 64) + 64, B, use_cuda_graph=False)
    long = [torch.randint(0, 32000, (ctx,), generator=g).tolist() for _ in range(B)]
    for i0 in range(0, B, 8):
        eng.step([(i, long[i], []) for i in range(i0, i0 + 8)])
    for _ in range(3):
        eng.step([(i, [7], [0]) for i in range(B)])
else:
    B, S = (8, 1024) if mode == 'prefill' else (2, 1024)
    eng = SequenceEngine(model, B * S + 64, B)
    p = [torch.randint(0, 32000, (S,), generator=g).tolist() for _ in range(B)]
    for _ in range(3):
        eng.step([(i, p[i], [S - 1]) for i in range(B)], list(range(B)))
torch.cuda.synchronize()
print('ok')
