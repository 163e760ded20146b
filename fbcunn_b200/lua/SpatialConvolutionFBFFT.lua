--[[
   nn.SpatialConvolutionFBFFT on top of libfbfftconv (B200, sm_100a).

   Drop-in for fbcunn/SpatialConvolutionFBFFT.lua: same class name, constructor
   arguments, nn.Module methods and weight / bias / gradWeight / gradBias layout, so a
   Torch7 model that builds the reference module runs unchanged.  The three passes are
   one C call each (include/fbfftconv.h) instead of the FFTWrapper / transposeMMFFI /
   bias-FFI sequence of the reference (fbcunn/SpatialConvolutionFBFFT.lua:102-354);
   there is no cudnn fallback: a failed pass raises a Lua error.

   Surface kept for the reference's callers:
     * nn.Module: updateOutput / updateGradInput / accGradParameters / backward / reset;
     * the per-pass implementations updateOutputFFTImpl(input, reuseList, metaData),
       updateGradInputFFTImpl(input, gradOutput, reuseList, metaData) and
       accGradParametersFFTImpl(input, gradOutput, scale, reuseList, metaData), which honour
       metaData.skipBias (fbcunn/SpatialConvolutionFBFFT.lua:172, :298);
     * the fields fbnn.SpatialConvolution reads and sets: printDebugLevel, cudnnDebug, success,
       autotuningPass, reportErrors, timeSteps (fbcunn/SpatialConvolutionFFT.lua:162-163, :259-268);
     * the second class name nn.SpatialConvolutionFBFFTGemm
       (fbcunn/SpatialConvolutionFBFFTGemm.lua:18-66) over the same native path;
     * nn.SpatialConvolutionFFTTiled (fbcunn/SpatialConvolutionFFTTiled.lua:265-365) over the
       library's tiled passes (fbfftconv_tiled_*), same constructor.
   Not kept: the class derives from nn.Module, not from the reference's nn.SpatialConvolutionFFT,
   so code that reaches into that base class's buffers, streams or FFTWrapper objects -- the
   reference's own SpatialConvolutionFFTTiled*.lua files do -- does not run on it.

   Requires LuaJIT (ffi), torch, cutorch.  Not executed by this repository's tests
   (no Lua toolchain there); the same C ABI is exercised from Python.
--]]
local ffi = require 'ffi'

ffi.cdef[[
typedef struct fbfftconv_handle fbfftconv_handle;
typedef struct fbfftconv_desc {
  int32_t batch, n_input_plane, n_output_plane;
  int32_t input_h, input_w, kernel_h, kernel_w;
  int32_t stride_h, stride_w, pad_h, pad_w;
  int32_t device;
  uint32_t flags;
} fbfftconv_desc;
int fbfftconv_create(const fbfftconv_desc* desc, fbfftconv_handle** out);
int fbfftconv_destroy(fbfftconv_handle* h);
int fbfftconv_fft_size(const fbfftconv_handle* h);
size_t fbfftconv_workspace_bytes(const fbfftconv_handle* h);
int fbfftconv_update_output(fbfftconv_handle* h, const float* input, const float* weight,
                            const float* bias, float* output, void* stream);
int fbfftconv_update_grad_input(fbfftconv_handle* h, const float* grad_output, const float* weight,
                                float* grad_input, void* stream);
int fbfftconv_acc_grad_parameters(fbfftconv_handle* h, const float* input, const float* grad_output,
                                  float* grad_weight, float* grad_bias, float scale, void* stream);
typedef struct fbfftconv_tiled fbfftconv_tiled;
int fbfftconv_tiled_create(const fbfftconv_desc* desc, int tile_h, int tile_w, fbfftconv_tiled** out);
int fbfftconv_tiled_destroy(fbfftconv_tiled* t);
fbfftconv_handle* fbfftconv_tiled_inner(fbfftconv_tiled* t);
int fbfftconv_tiled_update_output(fbfftconv_tiled* t, const float* input, const float* weight, const float* bias,
                                  float* output, void* stream);
int fbfftconv_tiled_update_grad_input(fbfftconv_tiled* t, const float* grad_output, const float* weight,
                                      float* grad_input, void* stream);
int fbfftconv_tiled_acc_grad_parameters(fbfftconv_tiled* t, const float* input, const float* grad_output,
                                        float* grad_weight, float* grad_bias, float scale, void* stream);
int fbfftconv_comm_unique_id(void* id128);
int fbfftconv_comm_init(fbfftconv_handle* h, const void* id128, int rank, int nranks);
const char* fbfftconv_last_error(void);
void* THCState_getCurrentStream(void* state);
]]

local lib_name = 'fbfftconv'
local lib_path = package.searchpath(lib_name, package.cpath)
local C = ffi.load(lib_path and lib_path or lib_name)

local FBFFTCONV_ACCUMULATE_GRADS = 1
local FBFFTCONV_REUSE_INPUT = 16
local FBFFTCONV_REUSE_OUTPUT = 32
local FBFFTCONV_REUSE_WEIGHT = 64

local SpatialConvolutionFBFFT, parent =
   torch.class('nn.SpatialConvolutionFBFFT', 'nn.Module')

SpatialConvolutionFBFFT.memoryReuseNone = "none"
SpatialConvolutionFBFFT.memoryReuseInput = "input"
SpatialConvolutionFBFFT.memoryReuseOutput = "output"
SpatialConvolutionFBFFT.memoryReuseWeight = "weight"
SpatialConvolutionFBFFT.memoryReuseAll = "all"

local function check(status)
   if status ~= 0 then
      error('fbfftconv: ' .. ffi.string(C.fbfftconv_last_error()))
   end
end

function SpatialConvolutionFBFFT:__init(nInputPlane, nOutputPlane, kW, kH, dW, dH,
                                        padLeft, padUp, memoryReusePolicy, numCudaStreams)
   parent.__init(self)
   for _, v in ipairs({nInputPlane, nOutputPlane, kW, kH}) do
      assert(torch.type(v) == 'number')
   end
   assert(memoryReusePolicy == nil or torch.type(memoryReusePolicy) == 'string' or
             torch.type(memoryReusePolicy) == 'table')
   assert(numCudaStreams == nil or torch.type(numCudaStreams) == 'number')
   self.nInputPlane, self.nOutputPlane = nInputPlane, nOutputPlane
   self.kW, self.kH = kW, kH
   self.dW, self.dH = dW or 1, dH or 1
   self.padLeft, self.padUp = padLeft or 0, padUp or 0
   self.padRight, self.padDown = self.padLeft, self.padUp
   assert(self.dH == 1, "fft only supports stride-1 convolutions atm")
   assert(self.dW == 1, "fft only supports stride-1 convolutions atm")
   assert(self.padUp < self.kH and self.padDown < self.kH and
             self.padLeft < self.kW and self.padRight < self.kW,
          "Padding must be smaller than kernel")
   self.fftImplementation = 'fbfft'
   self.memoryReusePolicy = memoryReusePolicy or SpatialConvolutionFBFFT.memoryReuseNone
   local function has(policy)
      local p = self.memoryReusePolicy
      if torch.type(p) == 'table' then
         for _, v in ipairs(p) do
            if v == policy or v == SpatialConvolutionFBFFT.memoryReuseAll then return true end
         end
         return false
      end
      return p == policy or p == SpatialConvolutionFBFFT.memoryReuseAll
   end
   self.reuseInputs = has(SpatialConvolutionFBFFT.memoryReuseInput)
   self.reuseOutputs = has(SpatialConvolutionFBFFT.memoryReuseOutput)
   self.reuseWeights = has(SpatialConvolutionFBFFT.memoryReuseWeight)
   self.numCudaStreams = numCudaStreams or 16
   self.accumulateGrads = false   -- reference behaviour: accGradParameters overwrites
   self.printDebugLevel = -1
   self.cudnnDebug = false
   self.success = true
   self.autotuningPass = false
   self.reportErrors = true
   self.timeSteps = { updateOutput = 0, updateGradInput = 0, accGradParameters = 0 }

   self.weight = torch.Tensor(nOutputPlane, nInputPlane, kH, kW)
   self.bias = torch.Tensor(nOutputPlane)
   self.gradWeight = torch.Tensor(nOutputPlane, nInputPlane, kH, kW)
   self.gradBias = torch.Tensor(nOutputPlane)
   self.output = torch.Tensor()
   self.gradInput = torch.Tensor()
   self:reset()
end

function SpatialConvolutionFBFFT:reset(stdv)
   if stdv then
      stdv = stdv * math.sqrt(3)
   else
      stdv = 1 / math.sqrt(self.kW * self.kH * self.nInputPlane)
   end
   self.weight:uniform(-stdv, stdv)
   self.bias:uniform(-stdv, stdv)
end

-- One native handle per (device, batch, image size); rebuilt when they change.
function SpatialConvolutionFBFFT:prepareSizeAndBuffers(input)
   assert(torch.type(input) == 'torch.CudaTensor', "CUDA support only!")
   assert(input:dim() == 4, "2D convolutions on 4D tensors atm")
   assert(input:isContiguous())
   local flags = (self.accumulateGrads and FBFFTCONV_ACCUMULATE_GRADS or 0)
      + (self.reuseInputs and FBFFTCONV_REUSE_INPUT or 0)
      + (self.reuseOutputs and FBFFTCONV_REUSE_OUTPUT or 0)
      + (self.reuseWeights and FBFFTCONV_REUSE_WEIGHT or 0)
   local key = string.format('%d:%d:%d:%d:%d', cutorch.getDevice(),
                             input:size(1), input:size(3), input:size(4), flags)
   if self.handleKey ~= key then
      self:cleanupBuffers()
      local desc = ffi.new('fbfftconv_desc', {
         input:size(1), self.nInputPlane, self.nOutputPlane,
         input:size(3), input:size(4), self.kH, self.kW,
         self.dH, self.dW, self.padUp, self.padLeft,
         cutorch.getDevice() - 1,
         flags})
      local out = ffi.new('fbfftconv_handle*[1]')
      check(C.fbfftconv_create(desc, out))
      self.handle = ffi.gc(out[0], C.fbfftconv_destroy)
      self.handleKey = key
      if self.comm then
         check(C.fbfftconv_comm_init(self.handle, self.comm.id, self.comm.rank, self.comm.nranks))
      end
   end
   return C.fbfftconv_fft_size(self.handle)
end

local function stream()
   return ffi.C.THCState_getCurrentStream(cutorch._state)
end

-- self.output / self.gradInput are made CUDA tensors once and only resized afterwards.
local function cudaResize(t, ...)
   if torch.type(t) ~= 'torch.CudaTensor' then t = torch.CudaTensor() end
   return t:resize(...)
end

function SpatialConvolutionFBFFT:updateOutputFFTImpl(input, reuseList, metaData)
   self:prepareSizeAndBuffers(input)
   local oH = input:size(3) + 2 * self.padUp - self.kH + 1
   local oW = input:size(4) + 2 * self.padLeft - self.kW + 1
   self.output = cudaResize(self.output, input:size(1), self.nOutputPlane, oH, oW)
   local bias = nil
   if not (metaData and metaData.skipBias) then bias = self.bias:data() end
   check(C.fbfftconv_update_output(self.handle, input:data(), self.weight:data(), bias,
                                   self.output:data(), stream()))
   return self.output
end

function SpatialConvolutionFBFFT:updateGradInputFFTImpl(input, gradOutput, reuseList, metaData)
   self:prepareSizeAndBuffers(input)
   assert(gradOutput:isContiguous())
   self.gradInput = cudaResize(self.gradInput, input:size())
   check(C.fbfftconv_update_grad_input(self.handle, gradOutput:data(), self.weight:data(),
                                       self.gradInput:data(), stream()))
   return self.gradInput
end

function SpatialConvolutionFBFFT:accGradParametersFFTImpl(input, gradOutput, scale, reuseList, metaData)
   self:prepareSizeAndBuffers(input)
   assert(gradOutput:isContiguous())
   local gradBias = nil
   if not (metaData and metaData.skipBias) then gradBias = self.gradBias:data() end
   check(C.fbfftconv_acc_grad_parameters(self.handle, input:data(), gradOutput:data(),
                                         self.gradWeight:data(), gradBias, scale or 1, stream()))
end

function SpatialConvolutionFBFFT:updateOutput(input)
   self.timeSteps.updateOutput = self.timeSteps.updateOutput + 1
   return self:updateOutputFFTImpl(input)
end

function SpatialConvolutionFBFFT:updateGradInput(input, gradOutput)
   self.timeSteps.updateGradInput = self.timeSteps.updateGradInput + 1
   return self:updateGradInputFFTImpl(input, gradOutput)
end

function SpatialConvolutionFBFFT:accGradParameters(input, gradOutput, scale)
   self.timeSteps.accGradParameters = self.timeSteps.accGradParameters + 1
   self:accGradParametersFFTImpl(input, gradOutput, scale)
end

function SpatialConvolutionFBFFT:backward(input, gradOutput, scale)
   self:updateGradInput(input, gradOutput)
   self:accGradParameters(input, gradOutput, scale)
   return self.gradInput
end

-- One process per GPU: `id` is the 128-byte value rank 0 got from
-- fbfftconv_comm_unique_id and shared with the other ranks.
function SpatialConvolutionFBFFT:attachCommunicator(id, rank, nranks)
   self.comm = {id = id, rank = rank, nranks = nranks}
   if self.handle then
      check(C.fbfftconv_comm_init(self.handle, id, rank, nranks))
   end
end

function SpatialConvolutionFBFFT:setReuseInputs(val) self.reuseInputs = val end
function SpatialConvolutionFBFFT:setReuseOutputs(val) self.reuseOutputs = val end
function SpatialConvolutionFBFFT:setReuseWeights(val) self.reuseWeights = val end

function SpatialConvolutionFBFFT:cleanupBuffers()
   self.handle = nil      -- ffi.gc destroys the native handle and its scratch
   self.handleKey = nil
   collectgarbage()
end

-- The reference's cgeam + cgemm variant (fbcunn/SpatialConvolutionFBFFTGemm.lua) under its own
-- class name: the spectra are bin-major from the transform on and the per-bin product is the same
-- tensor-core contraction, so the variant is this module.
local SpatialConvolutionFBFFTGemm, gemmParent =
   torch.class('nn.SpatialConvolutionFBFFTGemm', 'nn.SpatialConvolutionFBFFT')

function SpatialConvolutionFBFFTGemm:__init(...)
   gemmParent.__init(self, ...)
end

-- nn.SpatialConvolutionFFTTiled(nInputPlane, nOutputPlane, kW, kH, dW, dH, padLeft, padUp,
-- tileSizeW, tileSizeH, memoryReusePolicy, numCudaStreams), fbcunn/SpatialConvolutionFFTTiled.lua:265-365:
-- the same three passes on tiles of the image (overlap-save), done by the library's tiled entry
-- points; tile sizes default to 16 (:357-358).
local SpatialConvolutionFFTTiled, tiledParent =
   torch.class('nn.SpatialConvolutionFFTTiled', 'nn.SpatialConvolutionFBFFT')

function SpatialConvolutionFFTTiled:__init(nInputPlane, nOutputPlane, kW, kH, dW, dH,
                                           padLeft, padUp, tileSizeW, tileSizeH,
                                           memoryReusePolicy, numCudaStreams)
   assert(tileSizeW == nil or torch.type(tileSizeW) == 'number')
   assert(tileSizeH == nil or torch.type(tileSizeH) == 'number')
   tiledParent.__init(self, nInputPlane, nOutputPlane, kW, kH, dW, dH, padLeft, padUp,
                      memoryReusePolicy, numCudaStreams)
   self.tileSizeW = tileSizeW or 16
   self.tileSizeH = tileSizeH or 16
   assert(self.tileSizeH > self.kH - 1 and self.tileSizeW > self.kW - 1,
          "tile size must exceed the kernel size minus one")
end

function SpatialConvolutionFFTTiled:prepareSizeAndBuffers(input)
   assert(torch.type(input) == 'torch.CudaTensor', "CUDA support only!")
   assert(input:dim() == 4, "2D convolutions on 4D tensors atm")
   assert(input:isContiguous())
   local flags = (self.accumulateGrads and FBFFTCONV_ACCUMULATE_GRADS or 0)
      + (self.reuseInputs and FBFFTCONV_REUSE_INPUT or 0)
      + (self.reuseOutputs and FBFFTCONV_REUSE_OUTPUT or 0)
      + (self.reuseWeights and FBFFTCONV_REUSE_WEIGHT or 0)
   local key = string.format('%d:%d:%d:%d:%d', cutorch.getDevice(),
                             input:size(1), input:size(3), input:size(4), flags)
   if self.handleKey ~= key then
      self:cleanupBuffers()
      local desc = ffi.new('fbfftconv_desc', {
         input:size(1), self.nInputPlane, self.nOutputPlane,
         input:size(3), input:size(4), self.kH, self.kW,
         self.dH, self.dW, self.padUp, self.padLeft,
         cutorch.getDevice() - 1,
         flags})
      local out = ffi.new('fbfftconv_tiled*[1]')
      check(C.fbfftconv_tiled_create(desc, self.tileSizeH, self.tileSizeW, out))
      self.tiled = ffi.gc(out[0], C.fbfftconv_tiled_destroy)
      self.handle = C.fbfftconv_tiled_inner(self.tiled)   -- owned by the tiled handle
      self.handleKey = key
      if self.comm then
         check(C.fbfftconv_comm_init(self.handle, self.comm.id, self.comm.rank, self.comm.nranks))
      end
   end
end

function SpatialConvolutionFFTTiled:updateOutputFFTImpl(input, reuseList, metaData)
   self:prepareSizeAndBuffers(input)
   local oH = input:size(3) + 2 * self.padUp - self.kH + 1
   local oW = input:size(4) + 2 * self.padLeft - self.kW + 1
   self.output = cudaResize(self.output, input:size(1), self.nOutputPlane, oH, oW)
   local bias = nil
   if not (metaData and metaData.skipBias) then bias = self.bias:data() end
   check(C.fbfftconv_tiled_update_output(self.tiled, input:data(), self.weight:data(), bias,
                                         self.output:data(), stream()))
   return self.output
end

function SpatialConvolutionFFTTiled:updateGradInputFFTImpl(input, gradOutput, reuseList, metaData)
   self:prepareSizeAndBuffers(input)
   assert(gradOutput:isContiguous())
   self.gradInput = cudaResize(self.gradInput, input:size())
   check(C.fbfftconv_tiled_update_grad_input(self.tiled, gradOutput:data(), self.weight:data(),
                                             self.gradInput:data(), stream()))
   return self.gradInput
end

function SpatialConvolutionFFTTiled:accGradParametersFFTImpl(input, gradOutput, scale, reuseList, metaData)
   self:prepareSizeAndBuffers(input)
   assert(gradOutput:isContiguous())
   local gradBias = nil
   if not (metaData and metaData.skipBias) then gradBias = self.gradBias:data() end
   check(C.fbfftconv_tiled_acc_grad_parameters(self.tiled, input:data(), gradOutput:data(),
                                               self.gradWeight:data(), gradBias, scale or 1, stream()))
end

function SpatialConvolutionFFTTiled:cleanupBuffers()
   self.handle = nil
   self.tiled = nil       -- ffi.gc destroys the tiled handle and the untiled layer of the tiles with it
   self.handleKey = nil
   collectgarbage()
end
