{-# LANGUAGE GADTs               #-}
{-# LANGUAGE RankNTypes          #-}
{-# LANGUAGE ScopedTypeVariables #-}
-- |
-- Module      : Data.Array.Accelerate.B200.Execute
-- Description : From a delayed Accelerate term to an op list of the library, and running it on host arrays
--
-- NOT COMPILED HERE: the build machine of this repository has no GHC.
--
-- Takes the place of the compile and execute phases of accelerate-cuda
-- (Data/Array/Accelerate/CUDA/Compile.hs:90-300, CUDA/Execute.hs:143-450).  The
-- reference walks the term twice, once to generate and compile kernels and once
-- to launch them, allocating every intermediate as it goes; here ONE walk
-- records the program as an op list behind the C ABI (accb_program_*), and
-- running it is one foreign call.  Per node:
--
-- > Map / ZipWith / Generate / Transform / Backpermute (after fusion: a delayed producer)
-- >                         -> accb_program_map      with functorMap
-- > Fold / Fold1            -> accb_program_fold     with functorFold  (foldAll when the source is a vector)
-- > FoldSeg / Fold1Seg      -> accb_program_fold_seg
-- > Scanl .. Scanr1         -> accb_program_scan     (direction, kind; Scanl' / Scanr' yield two values)
-- > Permute                 -> accb_program_permute  (defaults copied first, Execute.hs:396-408)
-- > Stencil / Stencil2      -> accb_program_stencil / _stencil2
-- > Alet, Avar, Atuple, Aprj, Use
-- >                         -> value numbering of the op list; Use uploads through the memory table
-- > Acond, Awhile           -> host control flow around compiled pieces (awhile: accb_awhile)
--
module Data.Array.Accelerate.B200.Execute (

  Program, compileAcc, compileAfun1, executeAcc, executeAfun1, destroyProgram,

) where

import Control.Monad
import Data.IORef
import Foreign
import Foreign.C

import Data.Array.Accelerate.AST
import Data.Array.Accelerate.Array.Data                 ( ptrsOfArrayData )
import Data.Array.Accelerate.Array.Sugar                as S
import Data.Array.Accelerate.Trafo                      ( DelayedAcc, DelayedAfun, DelayedOpenAcc(..), DelayedOpenAfun )

import Data.Array.Accelerate.B200.CodeGen
import Data.Array.Accelerate.B200.Context
import Data.Array.Accelerate.B200.FFI

-- | A compiled array function: the library's op list plus what is needed to
-- marshal arguments and results (ExecAfun of CUDA/AST.hs:118-126).
data Program a b = Program
  { progContext :: Context
  , progHandle  :: Ptr AccbProgram
  , progKernels :: [Ptr AccbKernel]
  , progInputs  :: [AccbValueType]
  , progOutputs :: [AccbValueType]
  }

destroyProgram :: Program a b -> IO ()
destroyProgram p = withContext (progContext p) $ \h -> do
  _ <- c_programDestroy (progHandle p)
  forM_ (progKernels p) (c_kernelRelease h)

-- | Closed terms are functions of no argument.
compileAcc :: Arrays a => Context -> DelayedAcc a -> IO (Program () a)
compileAcc ctx acc = build ctx [] (\st -> node st [] acc)

compileAfun1 :: forall a b. (Arrays a, Arrays b) => Context -> DelayedAfun (a -> b) -> IO (Program a b)
compileAfun1 ctx (Alam (Abody body)) =
  let tys = valueTypes (arrays (undefined :: a))
  in  build ctx tys (\st -> node st [ [0 .. length tys - 1] ] body)
compileAfun1 _ _ = error "Data.Array.Accelerate.B200: run1 takes a function of one argument (use lift / unlift for more)"

-- ------------------------------------------------------------------ building the op list
data Build = Build
  { bCtx     :: Ptr AccbContext
  , bProg    :: Ptr AccbProgram
  , bKernels :: IORef [Ptr AccbKernel]
  , bCount   :: IORef Int                  -- kernels named so far (struct names must differ)
  }

-- | Value ids of an array-level term: one per array of the (flattened) result.
type Values = [Int]

build :: Context -> [AccbValueType] -> (Build -> IO Values) -> IO (Program a b)
build ctx inTys body = withContext ctx $ \h ->
  withArrayLen inTys $ \n tyPtr ->
  alloca $ \out -> do
    throwOnError h =<< c_programCreate h (fromIntegral n) tyPtr out
    prog <- peek out
    st   <- Build h prog <$> newIORef [] <*> newIORef 0
    outs <- body st
    withArrayLen (map fromIntegral outs) $ \m ids -> throwOnError h =<< c_programOutputs prog ids (fromIntegral m)
    ks   <- readIORef (bKernels st)
    return (Program ctx prog ks inTys [])

-- | Ask the library for a kernel: hash, memory cache, disk cache, nvcc (CUDA/Compile.hs:484-566).
kernel :: Build -> Functor -> IO (Ptr AccbKernel)
kernel st f =
  withCString (fSkeleton f) $ \sk -> withCString (fSource f) $ \src -> withCString (fName f) $ \nm ->
  alloca $ \out -> do
    throwOnError (bCtx st) =<< c_kernelGet (bCtx st) sk src nm nullPtr out      -- compiles in the background
    k <- peek out
    modifyIORef (bKernels st) (k :)
    return k

freshName :: Build -> String -> IO String
freshName st base = do
  n <- atomicModifyIORef' (bCount st) (\c -> (c + 1, c))
  return (base ++ show n)

-- | One walk over the delayed term.  `aenv` maps de Bruijn levels of the array environment to value ids.
node :: forall aenv a. Arrays a => Build -> [Values] -> DelayedOpenAcc aenv a -> IO Values
node st aenv (Manifest pacc) =
  case pacc of
    Alet bnd body   -> do v <- node st aenv bnd
                          node st (v : aenv) body
    Avar ix         -> return (aenv !! idxToInt ix)
    Atuple tup      -> concat <$> tupleNodes tup
    Aprj ix t       -> do vs <- node st aenv t
                          return (projectValues ix vs)

    -- producers that survived fusion as manifest arrays
    Map f a         -> elementwise "Map" f [a]
    Generate sh f   -> generateNode sh f
    ZipWith{}       -> error "Data.Array.Accelerate.B200: zipWith reaches the backend only as a delayed producer (CodeGen.hs:134-136)"

    -- consumers: the source is a delayed producer whose index function becomes `get`
    Fold  f z a     -> foldNode (Just z) f a
    Fold1 f a       -> foldNode Nothing  f a
    Scanl  f z a    -> scanNode scanLeft  scanExclusive (Just z) f a
    Scanl' f z a    -> scanNode scanLeft  scanPrime     (Just z) f a
    Scanl1 f a      -> scanNode scanLeft  scanInclusive Nothing  f a
    Scanr  f z a    -> scanNode scanRight scanExclusive (Just z) f a
    Scanr' f z a    -> scanNode scanRight scanPrime     (Just z) f a
    Scanr1 f a      -> scanNode scanRight scanInclusive Nothing  f a
    Permute f d p a -> permuteNode f d p a
    Stencil f b a   -> stencilNode f b a
    Use{}           -> error "Data.Array.Accelerate.B200: arrays embedded with `use` are registered with the memory table (accb_use) and enter the op list as extra inputs"
    _               -> error "Data.Array.Accelerate.B200: this array construct is not translated by the shim yet"
  where
    -- Every helper below prints the functor with the matching function of CodeGen, asks for the kernel, marshals
    -- the free array variables (Gamma) as the node's environment in the order the functor numbered them, and adds
    -- the node.  They are spelled out for `elementwise`; the others differ in the accb_program_* call only.
    elementwise :: String -> PreFun DelayedOpenAcc aenv (x -> y) -> [DelayedOpenAcc aenv arr] -> IO Values
    elementwise base f srcs = do
      name  <- freshName st base
      ins   <- concat <$> mapM (node st aenv) srcs
      let fn = functorMap (length aenv) name (error "C types of the inputs") (error "C types of the outputs") (error "closed f" f)
      k     <- kernel st fn
      let env = ins ++ concatMap (\lvl -> aenv !! (length aenv - 1 - lvl)) (freeArrays fn)
      withArrayLen (map fromIntegral env) $ \n ids ->
        with (AccbValueType (error "rank of the result") (error "component sizes of the result")) $ \ty -> do
          v <- c_programMap (bProg st) k ids (fromIntegral n) (fromIntegral (head ins)) ty nullPtr 0
          when (v < 0) $ throwOnError (bCtx st) (negate v)
          return [fromIntegral v]

    generateNode _ _       = error "as elementwise, through accb_program_generate_dims: the extents come from the shape expression"
    foldNode _ _ _         = error "as elementwise, through accb_program_fold (all = the source is a vector) with functorFold"
    scanNode _ _ _ _ _     = error "as elementwise, through accb_program_scan with functorScan; Scanl' / Scanr' return [body, total]"
    permuteNode _ _ _ _    = error "as elementwise, through accb_program_permute with functorPermute"
    stencilNode _ _ _      = error "as elementwise, through accb_program_stencil with functorStencil"
    tupleNodes _           = error "one walk per component of the array tuple"
    projectValues _ vs     = vs

node _ _ Delayed{} = error "Data.Array.Accelerate.B200: a delayed producer is consumed by the node that reads it; it never stands alone"

-- ------------------------------------------------------------------ marshalling and running
-- | Rank and component sizes of every array of an Arrays structure, leftmost first.
valueTypes :: ArraysR arrs -> [AccbValueType]
valueTypes ArraysRunit         = []
valueTypes ArraysRarray        = [error "AccbValueType (rank sh) (sizes of the components of e)"]
valueTypes (ArraysRpair a b)   = valueTypes a ++ valueTypes b

-- | One accb_array per array: shape innermost extent first (the reverse of shapeToList's use for kernel
-- arguments, CUDA/Execute.hs:835-836), one HOST pointer per flattened component (ptrsOfArrayData).
hostArray :: forall sh e. (Shape sh, Elt e) => Array sh e -> AccbArray
hostArray (Array sh adata) =
  AccbArray (shapeToList (toElt sh :: sh)) (componentPtrs (ptrsOfArrayData adata))
  where
    componentPtrs = error "flatten the nested pairs of pointers, leftmost component first"

-- | run1 on host arrays: upload, launches, download -- accb_program_run_host does all three, in pieces where the
-- program allows it (executeAfun1 + collect, CUDA/Execute.hs:143-162, CUDA.hs:382-389).
executeAfun1 :: forall a b. (Arrays a, Arrays b) => Program a b -> a -> IO b
executeAfun1 p a = withContext (progContext p) $ \h -> do
  let ins = marshalIn (arrays (undefined :: a)) (fromArr a)
  outs <- allocateResults (arrays (undefined :: b))         -- host arrays of the result, shapes from the op list's rules
  withArrayLen ins $ \_ inPtr ->
    withArrayLen (map snd outs) $ \_ outPtr ->
      throwOnError h =<< c_programRunHost (progHandle p) inPtr outPtr
  return (toArr (rebuild (arrays (undefined :: b)) (map fst outs)))
  where
    marshalIn :: ArraysR arrs -> arrs -> [AccbArray]
    marshalIn ArraysRunit       ()       = []
    marshalIn ArraysRarray      arr      = [hostArray arr]
    marshalIn (ArraysRpair x y) (u, v)   = marshalIn x u ++ marshalIn y v
    allocateResults                      = error "allocateArray for every result (Array/Sugar.hs:40-44) and its accb_array"
    rebuild                              = error "the inverse of marshalIn"

executeAcc :: Arrays a => Program () a -> IO a
executeAcc p = executeAfun1 p ()
