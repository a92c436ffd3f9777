"""Three decode steps at batch N then three at batch 1 on a 2-layer slice of the 27B config (8192-token contexts), between cudaProfilerStart/Stop."""
import os
import sys, dataclasses, numpy as np, torch
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))))
from rexl3_b200.models import dense
from rexl3_b200.engine.gpu_backend import DenseGpuBackend
from rexl3_b200.engine import Engine, Request
from rexl3_b200.sampling import GREEDY
cfg=dataclasses.replace(dense.CONFIGS['dense-27b'], n_layers=2, name='dense-27b-2L')
B=int(sys.argv[1]) if len(sys.argv)>1 else 64
P=8192
bps=(P+64)//64+2
m=dense.DenseGPU(cfg,num_pages=(B+1)*bps,max_rows=256,max_seqs=B+1,max_blocks_per_seq=bps,max_prefill_rows=P)
be=DenseGpuBackend(m,max_slots=B+1,use_graphs=False)
eng=Engine(be,None,window_rows=B,prefill_chunk=P,spec='none',prefill_policy='serial')
rng=np.random.default_rng(0)
eng.pause_decode=True
for i in range(B):
    eng.submit(Request(f's{i}',rng.integers(0,cfg.vocab,size=P).tolist(),40,GREEDY))
    while eng.seqs.get(f's{i}') is None or eng.seqs[f's{i}'].generated==0: eng.step()
eng.pause_decode=False
torch.cuda.synchronize()
torch.cuda.profiler.start()
for _ in range(3): eng.step()
torch.cuda.synchronize()
for i in range(1,B): eng.cancel(f's{i}')
for _ in range(3): eng.step()
torch.cuda.synchronize()
torch.cuda.profiler.stop()
print('ok')
