{-# LANGUAGE ForeignFunctionInterface #-}
{-# LANGUAGE RecordWildCards          #-}
-- |
-- Module      : Data.Array.Accelerate.B200.FFI
-- Description : Bindings to the C ABI of libaccb200.so (include/accb200.h)
--
-- NOT COMPILED HERE: the build machine of this repository has no GHC.  This
-- is the source a maintainer adds next to the library; it follows the
-- header declaration by declaration.
--
-- It takes the place of the calls into the @cuda@ package that
-- accelerate-cuda makes from Data/Array/Accelerate/CUDA/Execute.hs:930-982
-- (launchKernel), CUDA/Compile.hs:484-566 (loadData, nvcc), and
-- CUDA/Array/Prim.hs:159-391 (mallocArray, pokeArray, peekArray ...).
--
module Data.Array.Accelerate.B200.FFI (

  -- * Handles
  AccbContext, AccbKernel, AccbProgram, Stream,

  -- * Records
  AccbArray(..), AccbValueType(..), maxRank, maxComp,

  -- * Status
  Status, statusOK, throwOnError,

  -- * Contexts and kernels
  c_init, c_contextCreate, c_contextDestroy, c_contextSync, c_lastError,
  c_kernelGet, c_kernelWait, c_kernelRelease,

  -- * Single launches on device arrays
  c_map, c_foldAll, c_foldDim, c_foldSeg, c_scan, c_permuteDefaults, c_permute,
  c_stencil, c_stencil2, c_stencilIterate, c_stencilIterateFrom,

  -- * Memory table
  c_malloc, c_use, c_insertUnmanaged, c_withPtr, c_release, c_releaseAfter,
  c_peek, c_poke, c_free, c_reclaim,

  -- * Whole programs (the op list that stands for a compiled function)
  c_programCreate, c_programMap, c_programGenerate, c_programFold, c_programFoldSeg,
  c_programScan, c_programPermute, c_programStencil, c_programStencil2,
  c_programOutputs, c_programRun, c_programRunHost, c_programDestroy,

  -- * Constants of the header
  scanLeft, scanRight, scanExclusive, scanInclusive, scanPrime,
  boundaryClamp, boundaryMirror, boundaryWrap, boundaryConstant,

) where

import Control.Exception
import Control.Monad
import Foreign
import Foreign.C

data AccbContext
data AccbKernel
data AccbProgram
type Stream = Ptr ()
type Status = CInt

statusOK :: Status
statusOK = 0

maxRank, maxComp :: Int
maxRank = 4       -- ACCB_ARRAY_MAX_RANK
maxComp = 8       -- ACCB_ARRAY_MAX_COMP

-- | @struct accb_array@: rank, shape (innermost extent first), number of
-- components, one pointer per flattened tuple component (structure of arrays,
-- as CUDA/CodeGen/Base.hs:69-79 lays tuples out).
data AccbArray = AccbArray
  { arrShape :: [Int]          -- ^ innermost extent first
  , arrPtrs  :: [Ptr ()]
  }

instance Storable AccbArray where
  sizeOf    _ = 24 + 8 * maxComp   -- int rank; int shape[4]; int ncomp; void *ptr[8] (at offset 24)
  alignment _ = 8
  poke p AccbArray{..} = do
    pokeByteOff p 0 (fromIntegral (length arrShape) :: CInt)
    forM_ (zip [0 ..] (take maxRank (arrShape ++ repeat 0))) $ \(d, e) ->
      pokeByteOff p (4 + 4 * d) (fromIntegral e :: CInt)
    pokeByteOff p (4 + 4 * maxRank) (fromIntegral (length arrPtrs) :: CInt)
    forM_ (zip [0 ..] (take maxComp (arrPtrs ++ repeat nullPtr))) $ \(c, q) ->
      pokeByteOff p (24 + 8 * c) q
  peek p = do
    r  <- peekByteOff p 0 :: IO CInt
    sh <- forM [0 .. fromIntegral r - 1] $ \d -> (fromIntegral :: CInt -> Int) <$> peekByteOff p (4 + 4 * d)
    n  <- peekByteOff p (4 + 4 * maxRank) :: IO CInt
    ps <- forM [0 .. fromIntegral n - 1] $ \c -> peekByteOff p (24 + 8 * c)
    return (AccbArray sh ps)

-- | @struct accb_value_type@: what a program value looks like before it has a size.
data AccbValueType = AccbValueType
  { vtRank      :: Int
  , vtCompBytes :: [Int]       -- ^ bytes of every flattened component
  }

instance Storable AccbValueType where
  sizeOf    _ = 4 + 4 + 4 * maxComp
  alignment _ = 4
  poke p AccbValueType{..} = do
    pokeByteOff p 0 (fromIntegral vtRank :: CInt)
    pokeByteOff p 4 (fromIntegral (length vtCompBytes) :: CInt)
    forM_ (zip [0 ..] (take maxComp (vtCompBytes ++ repeat 0))) $ \(c, b) ->
      pokeByteOff p (8 + 4 * c) (fromIntegral b :: CInt)
  peek p = do
    r <- peekByteOff p 0 :: IO CInt
    n <- peekByteOff p 4 :: IO CInt
    b <- forM [0 .. fromIntegral n - 1] $ \c -> (fromIntegral :: CInt -> Int) <$> peekByteOff p (8 + 4 * c)
    return (AccbValueType (fromIntegral r) b)

-- | Every entry point returns a status; the message lives in the context
-- (the reference turns CUDA errors into exceptions, CUDA/State.hs:87-88).
throwOnError :: Ptr AccbContext -> Status -> IO ()
throwOnError ctx st =
  unless (st == statusOK) $ do
    msg <- peekCString =<< c_lastError ctx
    throwIO (ErrorCall ("accelerate-b200: " ++ msg))

scanLeft, scanRight, scanExclusive, scanInclusive, scanPrime :: CInt
scanLeft = 0; scanRight = 1; scanExclusive = 0; scanInclusive = 1; scanPrime = 2

boundaryClamp, boundaryMirror, boundaryWrap, boundaryConstant :: CInt
boundaryClamp = 0; boundaryMirror = 1; boundaryWrap = 2; boundaryConstant = 3

-- contexts: Context.create / destroy (CUDA/Context.hs:55-93), State.defaultContext
foreign import ccall unsafe "accb_init"            c_init           :: IO Status
foreign import ccall unsafe "accb_context_create"  c_contextCreate  :: CInt -> Ptr () -> Ptr (Ptr AccbContext) -> IO Status
foreign import ccall unsafe "accb_context_destroy" c_contextDestroy :: Ptr AccbContext -> IO Status
foreign import ccall safe   "accb_context_sync"    c_contextSync    :: Ptr AccbContext -> IO Status
foreign import ccall unsafe "accb_last_error"      c_lastError      :: Ptr AccbContext -> IO CString

-- kernel cache: build / compile / link (CUDA/Compile.hs:439-566, CUDA/Persistent.hs)
foreign import ccall safe "accb_kernel_get"
  c_kernelGet :: Ptr AccbContext -> CString {- skeleton -} -> CString {- functor source -}
              -> CString {- functor name -} -> CString {- nvcc flags or NULL -}
              -> Ptr (Ptr AccbKernel) -> IO Status
foreign import ccall safe   "accb_kernel_wait"    c_kernelWait    :: Ptr AccbContext -> Ptr AccbKernel -> IO Status
foreign import ccall unsafe "accb_kernel_release" c_kernelRelease :: Ptr AccbContext -> Ptr AccbKernel -> IO Status

-- one launch per skeleton: executeOp / foldCore / foldSegOp / scanOp / permuteOp / stencilOp
-- (CUDA/Execute.hs:264-450)
foreign import ccall safe "accb_map"
  c_map :: Ptr AccbContext -> Ptr AccbKernel -> Stream -> Ptr AccbArray -> CInt -> Ptr () -> CSize -> Ptr AccbArray -> IO Status
foreign import ccall safe "accb_fold_all"
  c_foldAll :: Ptr AccbContext -> Ptr AccbKernel -> Stream -> Ptr AccbArray -> CInt -> CLLong -> Ptr () -> CSize
            -> Ptr AccbArray -> IO Status
foreign import ccall safe "accb_fold_dim"
  c_foldDim :: Ptr AccbContext -> Ptr AccbKernel -> Stream -> Ptr AccbArray -> CInt -> CLLong -> CLLong -> Ptr () -> CSize
            -> Ptr AccbArray -> IO Status
foreign import ccall safe "accb_fold_seg"
  c_foldSeg :: Ptr AccbContext -> Ptr AccbKernel -> Stream -> Ptr AccbArray -> CInt -> CLLong -> CLLong -> Ptr CInt -> CLLong
            -> Ptr () -> CSize -> Ptr AccbArray -> IO Status
foreign import ccall safe "accb_scan"
  c_scan :: Ptr AccbContext -> Ptr AccbKernel -> Stream -> Ptr AccbArray -> CInt -> CLLong
         -> CInt {- direction -} -> CInt {- kind -} -> Ptr () -> CSize -> Ptr AccbArray -> Ptr AccbArray -> IO Status
foreign import ccall safe "accb_permute_defaults"
  c_permuteDefaults :: Ptr AccbContext -> Stream -> Ptr AccbArray -> Ptr AccbArray -> Ptr CInt -> IO Status
foreign import ccall safe "accb_permute"
  c_permute :: Ptr AccbContext -> Ptr AccbKernel -> Stream -> Ptr AccbArray -> CInt -> CLLong -> Ptr () -> CSize
            -> Ptr AccbArray -> IO Status
foreign import ccall safe "accb_stencil"
  c_stencil :: Ptr AccbContext -> Ptr AccbKernel -> Stream -> Ptr AccbArray -> CInt -> Ptr () -> CSize -> Ptr AccbArray -> IO Status
foreign import ccall safe "accb_stencil2"
  c_stencil2 :: Ptr AccbContext -> Ptr AccbKernel -> Stream -> Ptr AccbArray -> Ptr AccbArray -> CInt -> Ptr () -> CSize
             -> Ptr AccbArray -> IO Status
foreign import ccall safe "accb_stencil_iterate"
  c_stencilIterate :: Ptr AccbContext -> Ptr AccbKernel -> Stream -> Ptr AccbArray -> Ptr AccbArray -> CInt -> CInt
                   -> Ptr () -> CSize -> Ptr CInt -> IO Status
-- the same from a source that is only read; two applications per launch where the kernel has that form
foreign import ccall safe "accb_stencil_iterate_from"
  c_stencilIterateFrom :: Ptr AccbContext -> Ptr AccbKernel -> Stream -> Ptr AccbArray -> Ptr AccbArray -> Ptr AccbArray
                       -> CInt -> CInt -> Ptr () -> CSize -> Ptr CInt -> IO Status

-- memory table: malloc / withRemote / insertUnmanaged / free / reclaim (CUDA/Array/Remote.hs:91-202),
-- peek / poke (CUDA/Array/Prim.hs:189-391).  Keys are the hash of the host array's StableName.
foreign import ccall safe   "accb_malloc"           c_malloc          :: Ptr AccbContext -> Word64 -> CSize -> Ptr (Ptr ()) -> IO Status
foreign import ccall safe   "accb_use"              c_use             :: Ptr AccbContext -> Word64 -> Ptr () -> CSize -> Stream -> Ptr (Ptr ()) -> IO Status
foreign import ccall unsafe "accb_insert_unmanaged" c_insertUnmanaged :: Ptr AccbContext -> Word64 -> Ptr () -> CSize -> IO Status
foreign import ccall safe   "accb_with_ptr"         c_withPtr         :: Ptr AccbContext -> Word64 -> Ptr (Ptr ()) -> Ptr CSize -> IO Status
foreign import ccall unsafe "accb_release"          c_release         :: Ptr AccbContext -> Word64 -> IO Status
foreign import ccall unsafe "accb_release_after"    c_releaseAfter    :: Ptr AccbContext -> Word64 -> Stream -> IO Status
foreign import ccall safe   "accb_peek"             c_peek            :: Ptr AccbContext -> Word64 -> CSize -> Ptr () -> CSize -> Stream -> IO Status
foreign import ccall safe   "accb_poke"             c_poke            :: Ptr AccbContext -> Word64 -> CSize -> Ptr () -> CSize -> Stream -> IO Status
foreign import ccall safe   "accb_free"             c_free            :: Ptr AccbContext -> Word64 -> IO Status
foreign import ccall safe   "accb_reclaim"          c_reclaim         :: Ptr AccbContext -> IO Status

-- whole programs.  Node constructors return the id of the value they produce (negative: minus a status).
foreign import ccall unsafe "accb_program_create"
  c_programCreate :: Ptr AccbContext -> CInt -> Ptr AccbValueType -> Ptr (Ptr AccbProgram) -> IO Status
foreign import ccall unsafe "accb_program_map"
  c_programMap :: Ptr AccbProgram -> Ptr AccbKernel -> Ptr CInt -> CInt -> CInt -> Ptr AccbValueType -> Ptr () -> CSize -> IO CInt
foreign import ccall unsafe "accb_program_generate_dims"
  c_programGenerate :: Ptr AccbProgram -> Ptr AccbKernel -> Ptr CInt -> CInt -> CInt -> Ptr CInt -> Ptr CInt -> Ptr CInt
                    -> Ptr AccbValueType -> Ptr () -> CSize -> IO CInt
foreign import ccall unsafe "accb_program_fold"
  c_programFold :: Ptr AccbProgram -> Ptr AccbKernel -> Ptr CInt -> CInt -> CInt -> CInt -> Ptr () -> CSize -> Ptr AccbValueType -> IO CInt
foreign import ccall unsafe "accb_program_fold_seg"
  c_programFoldSeg :: Ptr AccbProgram -> Ptr AccbKernel -> Ptr CInt -> CInt -> CInt -> CInt -> Ptr () -> CSize -> Ptr AccbValueType -> IO CInt
foreign import ccall unsafe "accb_program_scan"
  c_programScan :: Ptr AccbProgram -> Ptr AccbKernel -> Ptr CInt -> CInt -> CInt -> CInt -> CInt -> Ptr () -> CSize
                -> Ptr AccbValueType -> IO CInt
foreign import ccall unsafe "accb_program_permute"
  c_programPermute :: Ptr AccbProgram -> Ptr AccbKernel -> Ptr CInt -> CInt -> CInt -> CInt -> Ptr AccbValueType -> IO CInt
foreign import ccall unsafe "accb_program_stencil"
  c_programStencil :: Ptr AccbProgram -> Ptr AccbKernel -> CInt -> CInt -> Ptr () -> CSize -> CInt -> Ptr AccbValueType -> IO CInt
foreign import ccall unsafe "accb_program_stencil2"
  c_programStencil2 :: Ptr AccbProgram -> Ptr AccbKernel -> CInt -> CInt -> CInt -> Ptr () -> CSize -> Ptr AccbValueType -> IO CInt
foreign import ccall unsafe "accb_program_outputs" c_programOutputs :: Ptr AccbProgram -> Ptr CInt -> CInt -> IO Status
foreign import ccall safe   "accb_program_run"
  c_programRun :: Ptr AccbProgram -> Stream -> Ptr AccbArray -> Ptr AccbArray -> IO Status
-- | run1 on host arrays: upload, launches and download, in pieces where the program allows it
foreign import ccall safe   "accb_program_run_host"
  c_programRunHost :: Ptr AccbProgram -> Ptr AccbArray -> Ptr AccbArray -> IO Status
foreign import ccall safe   "accb_program_destroy" c_programDestroy :: Ptr AccbProgram -> IO Status
