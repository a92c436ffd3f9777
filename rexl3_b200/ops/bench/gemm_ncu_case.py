"""A small fixed case of the EXL3 GEMM (gate_up shape, 64 and 2048 rows) for one ncu capture."""
import os
import sys, torch
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))))
from rexl3_b200.ops import kernels as K
dev='cuda'
k,n=5120,34816
tr=torch.randint(-32768,32767,(k//16,n//16,64),dtype=torch.int16,device=dev)
w=K.Exl3Weight(tr,torch.ones(k,dtype=torch.float16,device=dev),torch.ones(n,dtype=torch.float16,device=dev),None,'3inst')
status=K.new_status()
for rows in (64, 2048):
    splits=K.plan_splits(k,n,rows<=256)
    xr=(torch.randn(rows,k,device=dev)*0.5).to(torch.float16)
    part=torch.empty(splits*rows*n,dtype=torch.float32,device=dev)
    for _ in range(2): K.exl3_gemm(xr,w,part,splits,status)
    torch.cuda.synchronize()
K.check_status(status); print('ok')
