"""One 8192-token prefill on a 2-layer slice of the 27B config, between cudaProfilerStart/Stop."""
import os
import sys, dataclasses, numpy as np, torch
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))))
from rexl3_b200.models import dense
from rexl3_b200.engine.gpu_backend import DenseGpuBackend
from rexl3_b200.engine import Engine, Request
from rexl3_b200.sampling import GREEDY
cfg=dataclasses.replace(dense.CONFIGS['dense-27b'], n_layers=2, name='dense-27b-2L')
P=8192; bps=(P+64)//64+2
m=dense.DenseGPU(cfg,num_pages=3*bps,max_rows=256,max_seqs=3,max_blocks_per_seq=bps,max_prefill_rows=P)
be=DenseGpuBackend(m,max_slots=3,use_graphs=False)
eng=Engine(be,None,window_rows=2,prefill_chunk=P,spec='none',prefill_policy='serial')
rng=np.random.default_rng(0)
eng.pause_decode=True
def one(i):
    eng.submit(Request(f's{i}',rng.integers(0,cfg.vocab,size=P).tolist(),4,GREEDY))
    while eng.seqs.get(f's{i}') is None or eng.seqs[f's{i}'].generated==0: eng.step()
    torch.cuda.synchronize()
one(0)
e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
torch.cuda.profiler.start()
e0.record()
one(1)
e1.record()
torch.cuda.profiler.stop()
torch.cuda.synchronize()
print(f'2-layer 8192-token prefill: {e0.elapsed_time(e1):.2f} ms')
print('ok')
