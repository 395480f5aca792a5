"""Protocol models of the three persistent attention kernels (test infrastructure, CPU only).

Each role of a kernel (TMA producer, MMA issuers, compute / softmax warpgroups, D warps) is a
generator that yields the waits and arrivals it performs on the CTA's mbarriers, in the order of
autoresearch_b200/csrc/attn_fwd.cu, attn_bwd_dq.cu and attn_bwd.cu; `drive` runs the roles of one
CTA under random interleavings.  The barrier model has the hardware's parity semantics: a wait for
phase t succeeds whenever the barrier's open phase has the other parity, so it also "succeeds"
while phase t-1 is still open and blocks for ever once phase t+1 has completed - the two ways a
hand-shake can go wrong without any data race.  Over-arrival on a barrier raises.
"""
import random

class Bar:
    def __init__(s, name, count): s.name=name; s.count=count; s.pending=count; s.phase=0
    def arrive(s, n=1):
        s.pending-=n
        assert s.pending>=0, f"over-arrival on {s.name} phase {s.phase}"
        if s.pending==0: s.phase+=1; s.pending=s.count
    def done(s, parity): return (s.phase & 1) != parity
def fwd_item(item, B,H,T,W,n_qb):
    bh=B*H; qi=item//bh; q0=(n_qb-1-qi)*256
    it={'q0':q0,'act':[],'jlo_t':[],'jhi_t':[]}
    for X in range(2):
        qlo=q0+128*X; act=qlo<T
        klo=max(0,qlo-W) if W>0 else 0
        khi=min(qlo+127,T-1)
        it['act'].append(act); it['jlo_t'].append(klo>>7); it['jhi_t'].append((khi>>7) if act else (klo>>7)-1)
    it['jlo']=it['jlo_t'][0]; it['jhi']=it['jhi_t'][1] if it['act'][1] else it['jhi_t'][0]
    return it
def sched(k,c,G,n_items):
    base=k*G
    if base>=n_items: return -1
    idx=base+(G-1-c) if k&1 else base+c
    return idx if idx<n_items else -2
TABLE = None   # optional {cta: [items]}: an explicit item order instead of the kernels' static schedule
def items_of(c,G,n_items):
    if TABLE is not None:
        yield from TABLE.get(c, [])
        return
    k=0
    while True:
        it=sched(k,c,G,n_items); k+=1
        if it==-1: return
        if it==-2: continue
        yield it
def run_fwd(B,H,T,W,c,G=148):
    n_qb=(T+255)//256; n_items=n_qb*B*H
    bars={}
    def mk(n,cnt): bars[n]=Bar(n,cnt)
    mk('q_full',1); mk('q_free',2)
    for X in range(2):
        mk(f's_full{X}',1); mk(f'p0_{X}',1); mk(f'p1_{X}',1); mk(f'o_final{X}',1); mk(f'o_free{X}',1); mk(f'exp{X}',1)
        mk(f'stat{X}',1)
    for s in range(2):
        mk(f'k_full{s}',1); mk(f'k_empty{s}',2); mk(f'v_full{s}',1); mk(f'v_empty{s}',2)
    cnt={'exp0':0,'exp1':0}
    def tma():
        g=0;n=0
        for item in items_of(c,G,n_items):
            wi=fwd_item(item,B,H,T,W,n_qb)
            if n>0: yield ('wait','q_free',(n-1)&1)
            yield ('arrive','q_full',1)
            for j in range(wi['jlo'],wi['jhi']+1):
                s=g%2; par=((g//2)&1)^1
                yield ('wait',f'k_empty{s}',par); yield ('arrive',f'k_full{s}',1)
                yield ('wait',f'v_empty{s}',par); yield ('arrive',f'v_full{s}',1)
                g+=1
            n+=1
    def issuer(X):
        g0=0;gx=0;nx=0;n=0
        for item in items_of(c,G,n_items):
            wi=fwd_item(item,B,H,T,W,n_qb)
            n_kv=wi['jhi']-wi['jlo']+1
            if not wi['act'][X]:
                yield ('wait','q_full',n&1); yield ('arrive','q_free',1)
                for t in range(n_kv):
                    s_=(g0+t)%2; par=((g0+t)//2)&1
                    yield ('wait',f'k_full{s_}',par); yield ('wait',f'v_full{s_}',par)
                    yield ('arrive',f'k_empty{s_}',1); yield ('arrive',f'v_empty{s_}',1)
                g0+=n_kv; n+=1; continue
            jlo_x,jhi_x=wi['jlo_t'][X],wi['jhi_t'][X]
            sole=False
            yield ('wait','q_full',n&1)
            def st(j): return (g0+j-wi['jlo'])%2
            def pr(j): return ((g0+j-wi['jlo'])//2)&1
            def qk(j):
                s=st(j)
                yield ('wait',f'k_full{s}',pr(j))
                yield ('arrive',f's_full{X}',1); yield ('arrive',f'k_empty{s}',1)
                if sole: yield ('arrive',f'k_empty{s}',1)
                if j==jhi_x:
                    yield ('arrive','q_free',1)
                    if sole: yield ('arrive','q_free',1)
            for j in range(wi['jlo'],wi['jhi']+1):
                s=st(j)
                if not (jlo_x<=j<=jhi_x):
                    yield ('wait',f'k_full{s}',pr(j)); yield ('wait',f'v_full{s}',pr(j))
                    yield ('arrive',f'k_empty{s}',1); yield ('arrive',f'v_empty{s}',1); continue
                itx=j-jlo_x
                if itx==0:
                    yield from qk(j)
                yield ('wait',f'p0_{X}',(gx+itx)&1)
                yield ('wait',f'v_full{s}',pr(j))
                if itx==0 and nx>0: yield ('wait',f'o_free{X}',(nx-1)&1)
                yield ('wait',f'p1_{X}',(gx+itx)&1)
                if j==jhi_x: yield ('arrive',f'o_final{X}',1)
                yield ('arrive',f'v_empty{s}',1)
                if sole: yield ('arrive',f'v_empty{s}',1)
                if jlo_x<=j+1<=jhi_x and j+1<=wi['jhi']:
                    yield from qk(j+1)
            g0+=n_kv; gx+=jhi_x-jlo_x+1; nx+=1; n+=1
    def softmax(X):
        g_own=0;g_oth=0;nx=0;n=0
        for item in items_of(c,G,n_items):
            wi=fwd_item(item,B,H,T,W,n_qb)
            act_x=wi['act'][X]
            n_it=wi['jhi_t'][X]-wi['jlo_t'][X]+1 if act_x else 0
            Y=1-X
            n_other=wi['jhi_t'][Y]-wi['jlo_t'][Y]+1 if wi['act'][Y] else 0
            if not act_x:
                g_oth+=n_other; n+=1; continue
            for it in range(n_it):
                yield ('wait',f's_full{X}',(g_own+it)&1)
                if X==0:
                    if it==0 or it-1<n_other: yield ('cwait','exp1',g_oth+it)
                else:
                    if it<n_other: yield ('cwait','exp0',g_oth+it+1)
                yield ('arrive',f'p0_{X}',1)
                yield ('cinc',f'exp{X}',1)
                yield ('arrive',f'p1_{X}',1)
            # the row statistics go to the write-out warps; the previous item's have been read
            if nx>0: yield ('wait',f'o_free{X}',(nx-1)&1)
            yield ('arrive',f'stat{X}',1)
            g_own+=n_it; g_oth+=n_other; nx+=1; n+=1
    def writeout():
        nxe=[0,0]
        for item in items_of(c,G,n_items):
            wi=fwd_item(item,B,H,T,W,n_qb)
            for X in range(2):
                if not wi['act'][X]: continue
                yield ('wait',f'stat{X}',nxe[X]&1)
                yield ('wait',f'o_final{X}',nxe[X]&1)
                yield ('arrive',f'o_free{X}',1)
                nxe[X]+=1
    agents={'tma':tma(),'isA':issuer(0),'isB':issuer(1),'smA':softmax(0),'smB':softmax(1),'wo':writeout()}
    pending={k:None for k in agents}; done=set(); steps=0
    import random
    order=list(agents)
    while len(done)<len(agents):
        progress=False
        random.shuffle(order)
        for name in order:
            if name in done: continue
            # run this agent a random number of ops (to explore interleavings)
            for _ in range(random.randint(1,6)):
                op=pending[name]
                if op is None:
                    try: op=next(agents[name])
                    except StopIteration: done.add(name); progress=True; break
                if op[0]=='cwait':
                    if cnt[op[1]]>=op[2]: pending[name]=None; progress=True
                    else: pending[name]=op; break
                elif op[0]=='cinc':
                    cnt[op[1]]+=1; pending[name]=None; progress=True
                elif op[0]=='wait':
                    if bars[op[1]].done(op[2]): pending[name]=None; progress=True
                    else: pending[name]=op; break
                else:
                    bars[op[1]].arrive(op[2]); pending[name]=None; progress=True
        if not progress:
            print("DEADLOCK cta",c,{k:pending[k] for k in agents if k not in done},{b.name:(b.phase,b.pending) for b in bars.values()})
            return False
    return True

def drive(agents, bars, tag):
    pending={k:None for k in agents}; done=set(); order=list(agents)
    while len(done)<len(agents):
        progress=False; random.shuffle(order)
        for name in order:
            if name in done: continue
            for _ in range(random.randint(1,6)):
                op=pending[name]
                if op is None:
                    try: op=next(agents[name])
                    except StopIteration: done.add(name); progress=True; break
                if op[0]=='wait':
                    if bars[op[1]].done(op[2]): pending[name]=None; progress=True
                    else: pending[name]=op; break
                else:
                    bars[op[1]].arrive(op[2]); pending[name]=None; progress=True
        if not progress:
            print("DEADLOCK",tag,{k:pending[k] for k in agents if k not in done}); return False
    return True
def dkv_item(item,B,H,T,W):
    bh=B*H; kt=item//bh; row0=kt*128
    hi=min(T-1,row0+127+W) if W>0 else T-1
    hlo=row0//64; return dict(hlo=hlo,n_sub=hi//64-hlo+1)
def run_dkv(B,H,T,W,c,G=148):
    n_items=((T+127)//128)*B*H
    bars={}
    def mk(n,cnt): bars[n]=Bar(n,cnt)
    mk('x_full',1); mk('x_free',2); mk('acc_done',2); mk('acc_free',2)
    for s in range(4): mk(f'y_full{s}',1); mk(f'y_empty{s}',2)
    for i in range(2): mk(f'g_full{i}',2); mk(f'ready{i}',2)
    def tma():
        g=0;n=0
        for item in items_of(c,G,n_items):
            wi=dkv_item(item,B,H,T,W)
            if n>0: yield ('wait','x_free',(n-1)&1)
            yield ('arrive','x_full',1)
            for it in range(wi['n_sub']):
                s=g%4; yield ('wait',f'y_empty{s}',((g//4)&1)^1); yield ('arrive',f'y_full{s}',1); g+=1
            n+=1
    def issuer(I):
        g0=0;n=0
        for item in items_of(c,G,n_items):
            wi=dkv_item(item,B,H,T,W); ns=wi['n_sub']
            def acc(it,gg):
                s=gg%4; bf=gg&1
                yield ('wait',f'ready{bf}',(gg>>1)&1)
                if it==0 and n>0: yield ('wait','acc_free',(n-1)&1)
                yield ('arrive',f'y_empty{s}',1)
            yield ('wait','x_full',n&1)
            for it in range(ns):
                gg=g0+it; s=gg%4; bf=gg&1
                yield ('wait',f'y_full{s}',(gg//4)&1)
                yield ('arrive',f'g_full{bf}',1)
                if it==ns-1: yield ('arrive','x_free',1)
                if it>0: yield from acc(it-1,gg-1)
            yield from acc(ns-1,g0+ns-1)
            yield ('arrive','acc_done',1)
            g0+=ns; n+=1
    def compute(wg):
        g0=0;n=0
        for item in items_of(c,G,n_items):
            wi=dkv_item(item,B,H,T,W); ns=wi['n_sub']
            for it in range(ns):
                gg=g0+it; bf=gg&1; s=gg%4
                yield ('wait',f'y_full{s}',(gg//4)&1)
                yield ('wait',f'g_full{bf}',(gg>>1)&1)
                yield ('arrive',f'ready{bf}',1)
            g0+=ns
            yield ('wait','acc_done',n&1)
            yield ('arrive','acc_free',1)
            n+=1
    return drive({'tma':tma(),'is0':issuer(0),'is1':issuer(1),'wg0':compute(0),'wg1':compute(1)},bars,f"dkv cta {c}")
def dq_item(item,B,H,T,W,n_qt):
    bh=B*H; qi=item//bh; row0=(n_qt-1-qi)*128
    klo=max(0,row0-W) if W>0 else 0; khi=min(row0+127,T-1)
    return dict(n_it=(khi>>7)-(klo>>7)+1, jlo=klo>>7, row0=row0)
def run_dq(B,H,T,W,c,fuse,G=148):
    n_qt=(T+127)//128; n_items=n_qt*B*H
    bars={}
    def mk(n,cnt): bars[n]=Bar(n,cnt)
    mk('x_full',1); mk('x_free',2); mk('g_full',2); mk('g_free',4)
    for i in range(2): mk(f'ready{i}',4); mk(f'ds_free{i}',1)
    mk('acc_done',1); mk('acc_free',4); mk('epi_free',4)
    for s in range(3): mk(f'k_full{s}',1); mk(f'k_empty{s}',2)
    for s in range(2): mk(f'v_full{s}',1); mk(f'v_empty{s}',1); mk(f'd_ready{s}',1); mk(f'd_taken{s}',4)
    def tma():
        g=0;n=0;epi_item=-1;epi_slot=0
        for item in items_of(c,G,n_items):
            wi=dq_item(item,B,H,T,W,n_qt)
            if n>0: yield ('wait','x_free',(n-1)&1)
            yield ('arrive','x_full',1)
            for it in range(wi['n_it']):
                sk=g%3; sv=g%2
                yield ('wait',f'k_empty{sk}',((g//3)&1)^1); yield ('arrive',f'k_full{sk}',1)
                yield ('wait',f'v_empty{sv}',((g//2)&1)^1)
                if epi_item>=0 and (sv==epi_slot or it==wi['n_it']-1):
                    yield ('wait','epi_free',epi_item&1); epi_item=-1
                yield ('arrive',f'v_full{sv}',1)
                g+=1
            epi_item=n; epi_slot=(g-1)%2; n+=1
    def issuer(I):
        g=0;n=0
        for item in items_of(c,G,n_items):
            wi=dq_item(item,B,H,T,W,n_qt)
            yield ('wait','x_full',n&1)
            for it in range(wi['n_it']):
                s=g%3 if I==0 else g%2
                yield ('wait',(f'k_full{s}' if I==0 else f'v_full{s}'),(g//(3 if I==0 else 2))&1)
                if g>0: yield ('wait','g_free',(g-1)&1)
                yield ('arrive','g_full',1)
                yield ('arrive',(f'k_empty{s}' if I==0 else f'v_empty{s}'),1)
                if it==wi['n_it']-1: yield ('arrive','x_free',1)
                g+=1
            n+=1
    def dqiss():
        g=0;n=0
        for item in items_of(c,G,n_items):
            wi=dq_item(item,B,H,T,W,n_qt)
            for it in range(wi['n_it']):
                s=g%3
                yield ('wait',f'ready{g&1}',(g>>1)&1)
                if it==0 and n>0: yield ('wait','acc_free',(n-1)&1)
                yield ('arrive',f'ds_free{g&1}',1); yield ('arrive',f'k_empty{s}',1)
                g+=1
            yield ('arrive','acc_done',1); n+=1
    def dwarps():
        n=0
        for item in items_of(c,G,n_items):
            if n>1: yield ('wait',f'd_taken{n&1}',((n>>1)-1)&1)
            yield ('arrive',f'd_ready{n&1}',1); n+=1
    def two_term(wi,it):
        # tiles that can hold queries with fewer than 16 visible keys keep a residual in the other dS buffer
        kb=(wi['jlo']+it)*128; row0=wi['row0']
        if 0<W<15: return kb+127>row0 or kb<row0+127-W
        return row0==0 and kb==0
    def compute(wg):
        g=0;n=0;prev_two=False
        for item in items_of(c,G,n_items):
            wi=dq_item(item,B,H,T,W,n_qt)
            for it in range(wi['n_it']):
                yield ('wait','g_full',g&1)
                yield ('arrive','g_free',1)
                if it==0 and fuse:
                    yield ('wait',f'd_ready{n&1}',(n>>1)&1); yield ('arrive',f'd_taken{n&1}',1)
                two=two_term(wi,it)
                if g>1: yield ('wait',f'ds_free{g&1}',((g>>1)-1)&1)
                if g>0 and (prev_two or two): yield ('wait',f'ds_free{(g-1)&1}',((g-1)>>1)&1)
                yield ('arrive',f'ready{g&1}',1)
                prev_two=two
                g+=1
            yield ('wait','acc_done',n&1); yield ('arrive','acc_free',1); yield ('arrive','epi_free',1)
            n+=1
    ag={'tma':tma(),'isS':issuer(0),'isP':issuer(1),'isQ':dqiss()}
    for wg in range(4): ag[f'wg{wg}']=compute(wg)
    if fuse: ag['dw']=dwarps()
    return drive(ag,bars,f"dq cta {c} fuse {fuse}")
