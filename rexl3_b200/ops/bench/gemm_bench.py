"""CUDA-event timings of the EXL3 GEMM at the 27B config's five matrix shapes (median of 12, weights rotated over several copies)."""
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))))
import json, torch
from rexl3_b200.ops import kernels as K
torch.manual_seed(0)
dev='cuda'
def mk(k,n,bits=4,copies=4):
    ws=[]
    for c in range(copies):
        tr=torch.randint(-32768,32767,(k//16,n//16,int(16*bits)),dtype=torch.int16,device=dev)
        ws.append(K.Exl3Weight(tr,torch.ones(k,dtype=torch.float16,device=dev),torch.ones(n,dtype=torch.float16,device=dev),None,'3inst'))
    return ws
status=K.new_status()
shapes=dict(qkv=(5120,7168),o=(5120,5120),gate_up=(5120,34816),down=(17408,5120),lm_head=(5120,151936))
res={}
for name,(k,n) in shapes.items():
    ws=mk(k,n,copies=2 if name=='lm_head' else 6)
    for rows in (1,16,64,256,2048,8192):
        if name=='lm_head' and rows>256: continue
        decode= rows<=256
        splits=K.plan_splits(k,n,decode)
        xr=(torch.randn(rows,k,device=dev)*0.5).to(torch.float16)
        part=torch.empty(splits*rows*n,dtype=torch.float32,device=dev)
        for w in ws[:3]: K.exl3_gemm(xr,w,part,splits,status)
        torch.cuda.synchronize(); K.check_status(status)
        iters=12
        evs=[(torch.cuda.Event(enable_timing=True),torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
        for i in range(iters):
            evs[i][0].record(); K.exl3_gemm(xr,ws[i%len(ws)],part,splits,status); evs[i][1].record()
        torch.cuda.synchronize(); K.check_status(status)
        ts=sorted(a.elapsed_time(b) for a,b in evs)
        t=ts[len(ts)//2]
        wbytes=k*n/2
        fl=2*rows*k*n
        res[f'{name}_r{rows}']=dict(ms=t,splits=splits,GBs=wbytes/t/1e6,TFLOPs=fl/t/1e9)
        print(name,rows,'splits',splits,f'{t*1000:.1f} us  {wbytes/t/1e6:.0f} GB/s weights  {fl/t/1e9:.1f} TFLOP/s',flush=True)
    del ws; torch.cuda.empty_cache()
print(json.dumps(res))
