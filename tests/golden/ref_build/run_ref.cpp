// probe-only driver: reference LLamaModel on the CPU device, tiny random .bin
#include "model/llama3.h"
#include "scheduler/scheduler.h"
#include <cstdio>
#include "cpu/rope_kernel.h"
// "rope <head_size> <positions> <theta> <out>": the reference's sine/cosine tables for a theta of the caller's choice
// (its table function takes theta as an argument; only its model code fixes the value)
static int rope_tables(char**argv){ int hs=atoi(argv[2]), n=atoi(argv[3]); float theta=atof(argv[4]);
  std::vector<float> sn((size_t)hs*n), cs((size_t)hs*n); kernel::sin_cos_cache_calc_cpu(hs,n,sn.data(),cs.data(),theta);
  FILE* o=fopen(argv[5],"wb"); fwrite(sn.data(),4,sn.size(),o); fwrite(cs.data(),4,cs.size(),o); fclose(o); return 0; }
int main(int argc,char**argv){
  if(argc>5 && std::string(argv[1])=="rope") return rope_tables(argv);
  const char* bin=argv[1]; int max_seq=atoi(argv[2]);
  auto m=std::make_shared<model::LLamaModel>(base::TokenizerType::kEncodeSpe,"tok",bin,false);
  auto st=m->init(base::DeviceType::kDeviceCPU); if(!st){printf("init failed %d %s\n",int(st),st.get_err_msg().c_str());return 1;}
  printf("L=%d kv_dim=%d dim=%d vocab=%d seq=%d\n",m->layer_num(),m->kv_dim(),m->hidden_dim(),m->vocab_size(),m->seq_len());
  // direct forward_batch, continuous layout [L, slots, kv_dim, max_seq]
  auto a=base::CPUDeviceAllocatorFactory::get_instance();
  int L=m->layer_num(), kvd=m->kv_dim(), V=m->vocab_size();
  tensor::Tensor kc(base::DataType::kDataTypeFp32,L,1,kvd,max_seq,true,a), vc(base::DataType::kDataTypeFp32,L,1,kvd,max_seq,true,a);
  std::vector<int> prompt; FILE* f=fopen(argv[3],"r"); int t; while(fscanf(f,"%d",&t)==1) prompt.push_back(t); fclose(f);
  int n=prompt.size();
  tensor::Tensor ids(base::DataType::kDataTypeInt32,n,true,a), pos(base::DataType::kDataTypeInt32,n,true,a), bt(base::DataType::kDataTypeInt32,n,1,true,a), logits(base::DataType::kDataTypeFp32,n,V,true,a);
  for(int i=0;i<n;i++){ids.ptr<int32_t>()[i]=prompt[i];pos.ptr<int32_t>()[i]=i;bt.ptr<int32_t>()[i]=0;}
  st=m->forward_batch(ids,pos,bt,kc,vc,logits,true); if(!st){printf("fwd failed\n");return 1;}
  FILE* o=fopen(argv[4],"wb"); fwrite(logits.ptr<float>(),4,(size_t)n*V,o); fclose(o);
  // scheduler run: greedy generation, slot-mode (block_size = max_seq)
  scheduler::Scheduler s(m,4,max_seq,8,max_seq); s.add_request(prompt); std::vector<int> p2(prompt.begin(),prompt.begin()+3); s.add_request(p2);
  while(!s.all_finished()) s.step();
  for(auto& q: s.get_finished()){ printf("SEQ %d gen:",q.id); for(int g: q.generated_tokens) printf(" %d",g); printf("\n"); }
  return 0; }
