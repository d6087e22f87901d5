"""Random shapes, strides, dtypes and emulated SM counts through the four modes of the decode kernel on CPU threads,
each compared bit for bit with the oracle (int8 rows, fused quantizer, published row maxima) or with the definition
of the digit-plane path.  TEST INFRASTRUCTURE ONLY.

    python -m tests.simt.fuzz [seed] [seconds]

Prints one JSON line per failing case and a summary line."""

import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import numpy as np
import oracle
from tests.simt import harness as H
_planes_reference = H.planes_reference
L=H.lib()
rng=np.random.default_rng(int(sys.argv[1]) if len(sys.argv)>1 else 0)
budget=float(sys.argv[2]) if len(sys.argv)>2 else 600
t0=time.time(); n_cases=0; fails=[]
while time.time()-t0 < budget:
    m=int(rng.integers(1,17)); k=int(rng.choice([rng.integers(1,64), rng.integers(64,1200), rng.integers(1200,9000)]))
    n=int(rng.integers(1,140)); sms=int(rng.integers(1,9)); dtype=int(rng.choice([H.F32,H.BF16,H.F16])); mode=int(rng.integers(0,4))
    H.set_sm_count(sms)
    codes=rng.integers(-1,2,(n,k)).astype(np.int8); scale=(rng.random(n)*0.5+0.05).astype(np.float32)
    bias=rng.standard_normal(n).astype(np.float32) if rng.random()<0.5 else None
    tiled=H.retile(oracle.pack_transposed(codes),k)
    ld=k+int(rng.choice([0,4,8,3]))
    x=rng.standard_normal((m,ld)).astype(np.float32)*float(10.0**rng.integers(-2,2))
    xb=H.to_bits(x,dtype); x32=H.from_bits(np.ascontiguousarray(xb[:,:k]),dtype)
    y=H.empty_out((m,n),dtype)
    case=dict(m=m,k=k,n=n,sms=sms,dtype=dtype,mode=mode,ld=ld,bias=bias is not None)
    try:
        if mode==0:
            q,sx=oracle.act_quant(x32); acc=np.empty((m,n),np.int32)
            H.check(L.bt_gemv_tiled_i8(H.ptr(q),H.ptr(sx),m,k,H.ptr(tiled),n,H.ptr(scale),H.ptr(bias),H.ptr(y),dtype,n,H.ptr(acc),0,None))
            ref=oracle.gemm_i32(q,codes); ok=np.array_equal(acc,ref) and np.array_equal(y,H.to_bits(oracle.epilogue(ref,sx,scale,bias),dtype))
        elif mode==1:
            H.check(L.bt_gemv_tiled(H.ptr(xb),dtype,m,k,ld,H.ptr(tiled),n,H.ptr(scale),H.ptr(bias),H.ptr(y),dtype,n,None,None,None,0,None))
            q,sx=oracle.act_quant(x32); ok=np.array_equal(y,H.to_bits(oracle.epilogue(oracle.gemm_i32(q,codes),sx,scale,bias),dtype))
        elif mode==2:
            amax=np.zeros((m,8),np.uint32); mx=np.abs(x32).max(axis=1).astype(np.float32)
            amax[np.arange(m),rng.integers(0,8,m)]=mx.view(np.uint32)
            out_amax=np.zeros((m,8),np.uint32); cols=int(rng.integers(1,n+1))
            H.check(L.bt_gemv_tiled_chained(H.ptr(xb),dtype,m,k,ld,H.ptr(tiled),n,H.ptr(scale),H.ptr(bias),H.ptr(y),dtype,n,H.ptr(amax),H.ptr(out_amax),cols,0,None))
            q,sx=oracle.act_quant(x32); yr=H.to_bits(oracle.epilogue(oracle.gemm_i32(q,codes),sx,scale,bias),dtype)
            want=np.abs(H.from_bits(np.ascontiguousarray(yr[:,:cols]),dtype)).max(axis=1).astype(np.float32)
            ok=np.array_equal(y,yr) and np.array_equal(out_amax.max(axis=1).view(np.float32),want)
        else:
            if k>65536: continue
            H.check(L.bt_gemv_tiled_float(H.ptr(xb),dtype,m,k,ld,H.ptr(tiled),n,H.ptr(scale),H.ptr(bias),H.ptr(y),dtype,n,0,None))
            ok=np.array_equal(y,H.to_bits(_planes_reference(x32,codes,scale,bias),dtype))
        if H.device_status()!=0: ok=False
    except Exception as e:
        ok=False; case['exc']=str(e)[:200]
    n_cases+=1
    if not ok:
        fails.append(case); print("FAIL",json.dumps(case),flush=True)
print(json.dumps({"cases":n_cases,"fails":len(fails),"seconds":time.time()-t0}))
