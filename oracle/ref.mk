# Builds the UNMODIFIED reference library (srose69/nvfp4effma) for sm_100 from its own sources where they
# lie (REF, read-only), into oracle/_ref/ only.  Test infrastructure: the result pins the CPU oracle against
# the reference's own CUDA-core kernels on a B200 (tests/test_ref_pin_gpu.py) and is never linked into the product.
# The object list restates the reference Makefile's instance matrix (Makefile:46-54 there): one object per
# kernel instance, selected by -D macros.
ifndef REF
$(error REF is not set: make -f oracle/ref.mk REF=<directory of the reference's sources>)
endif
OUT  ?= oracle/_ref
NVCC ?= /usr/local/cuda/bin/nvcc
FLAGS = -O3 -Xptxas -O3 -std=c++14 -Xcompiler -ffp-contract=off,-fPIC -gencode arch=compute_100,code=sm_100
O = $(OUT)/obj

F_ALL = 0 1 2 3 4 5 6 7 8 9 10 11 12 13 14 15
F_A   = 0 1 2 3
EX    = 1 2 3 4 5
GEMV_IDS = 0 2
GEMM_IDS = 0 1
w = $(word $(1),$(subst _, ,$(2)))

INST = $(foreach i,$(GEMV_IDS),$(foreach t,1 4,$(foreach x,$(EX),gemvx_$(i)_$(t)_$(x)))) \
       $(foreach x,$(EX),$(foreach i,$(GEMM_IDS),gemmx_$(i)_1_$(x)) gemmx_0_4_$(x) dp4ax_$(x)) \
       $(foreach x,$(EX),gtcx_4_$(x) gtcx_1_$(x) tcx_4_$(x) tcx_1_$(x)) \
       $(foreach i,$(GEMV_IDS),$(foreach f,$(F_ALL),gemv_$(i)_0_$(f)) $(foreach t,1 2 3 4,$(foreach f,$(F_A),gemv_$(i)_$(t)_$(f)))) \
       $(foreach i,$(GEMM_IDS),$(foreach t,1 2 3,$(foreach f,$(F_A),gemm_$(i)_$(t)_$(f)))) \
       $(foreach f,$(F_ALL),gemm_0_0_$(f) dp4a_0_$(f)) $(foreach f,$(F_A),gemm_0_4_$(f) dp4a_4_$(f)) \
       $(foreach f,0 2 8 10,tc_0_$(f)) $(foreach f,0 2,tc_4_$(f) tc_1_$(f)) \
       $(foreach f,0 2 4 6 8 10 12 14 16 18 24 26,gtc_0_$(f)) $(foreach f,0 2,gtc_4_$(f) gtc_1_$(f)) \
       $(foreach t,1 2 3,$(foreach c,0 1,quant_$(t)_$(c)_1 quant_$(t)_$(c)_16))
OBJS = $(O)/nvfp4effma.o $(O)/gemm_nvfp4effma.o $(O)/gemv_nvfp4effma.o $(O)/tc_image.o $(foreach i,$(INST),$(O)/inst_$(i).o)

all: $(OUT)/libnvfp4effma_ref.so
$(OUT)/libnvfp4effma_ref.so: $(OBJS)
	$(NVCC) -shared -o $@ $^ -lcudart
$(O):
	mkdir -p $@
$(O)/nvfp4effma.o: $(REF)/src/nvfp4effma.cu | $(O)
	$(NVCC) $(FLAGS) -c -o $@ $<
$(O)/gemm_nvfp4effma.o: $(REF)/src/gemm_nvfp4effma.cu | $(O)
	$(NVCC) $(FLAGS) -c -o $@ $<
$(O)/gemv_nvfp4effma.o: $(REF)/src/gemv_nvfp4effma.cu | $(O)
	$(NVCC) $(FLAGS) -c -o $@ $<
$(O)/tc_image.o: $(REF)/src/tensors/image.cu | $(O)
	$(NVCC) $(FLAGS) -c -o $@ $<
$(O)/inst_gemmx_%.o: $(REF)/src/gemm_nvfp4effma_inst.cu | $(O)
	$(NVCC) $(FLAGS) -DNVFP4A_ID=$(call w,1,$*) -DNVFP4A_TB=$(call w,2,$*) -DNVFP4A_EX=$(call w,3,$*) -c -o $@ $<
$(O)/inst_dp4ax_%.o: $(REF)/src/gemm_dp4a_inst.cu | $(O)
	$(NVCC) $(FLAGS) -DNVFP4A_EX=$* -c -o $@ $<
$(O)/inst_gemm_%.o: $(REF)/src/gemm_nvfp4effma_inst.cu | $(O)
	$(NVCC) $(FLAGS) -DNVFP4A_ID=$(call w,1,$*) -DNVFP4A_TB=$(call w,2,$*) -DNVFP4A_F=$(call w,3,$*) -c -o $@ $<
$(O)/inst_dp4a_%.o: $(REF)/src/gemm_dp4a_inst.cu | $(O)
	$(NVCC) $(FLAGS) -DNVFP4A_TB=$(call w,1,$*) -DNVFP4A_F=$(call w,2,$*) -c -o $@ $<
$(O)/inst_tcx_%.o: $(REF)/src/tensors/gemm_tc_inst.cu | $(O)
	$(NVCC) $(FLAGS) -DNVFP4A_TB=$(call w,1,$*) -DNVFP4A_EX=$(call w,2,$*) -c -o $@ $<
$(O)/inst_tc_%.o: $(REF)/src/tensors/gemm_tc_inst.cu | $(O)
	$(NVCC) $(FLAGS) -DNVFP4A_TB=$(call w,1,$*) -DNVFP4A_F=$(call w,2,$*) -c -o $@ $<
$(O)/inst_gtcx_%.o: $(REF)/src/tensors/gemv_tc_inst.cu | $(O)
	$(NVCC) $(FLAGS) -DNVFP4A_TB=$(call w,1,$*) -DNVFP4A_EX=$(call w,2,$*) -c -o $@ $<
$(O)/inst_gtc_%.o: $(REF)/src/tensors/gemv_tc_inst.cu | $(O)
	$(NVCC) $(FLAGS) -DNVFP4A_TB=$(call w,1,$*) -DNVFP4A_F=$(call w,2,$*) -c -o $@ $<
$(O)/inst_quant_%.o: $(REF)/src/quant_nvfp4effma_inst.cu | $(O)
	$(NVCC) $(FLAGS) -DNVFP4A_QT=$(call w,1,$*) -DNVFP4A_QCOL=$(call w,2,$*) -DNVFP4A_QTILE=$(call w,3,$*) -c -o $@ $<
$(O)/inst_gemvx_%.o: $(REF)/src/gemv_nvfp4effma_inst.cu | $(O)
	$(NVCC) $(FLAGS) -DNVFP4A_ID=$(call w,1,$*) -DNVFP4A_TX=$(call w,2,$*) -DNVFP4A_F=0 -DNVFP4A_EX=$(call w,3,$*) -c -o $@ $<
$(O)/inst_gemv_%.o: $(REF)/src/gemv_nvfp4effma_inst.cu | $(O)
	$(NVCC) $(FLAGS) -DNVFP4A_ID=$(call w,1,$*) -DNVFP4A_TX=$(call w,2,$*) -DNVFP4A_F=$(call w,3,$*) -c -o $@ $<
.PHONY: all
